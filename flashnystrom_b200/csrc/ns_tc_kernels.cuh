// Newton-Schulz pseudoinverse on the sm_100a tensor cores with FP32-equivalent arithmetic.
//
// Every 64 x 64 FP32 matrix of the iteration is kept in shared memory as three bf16 tiles
// x = x0 + x1 + x2 (each term the bf16 rounding of what the previous terms left over: 24
// significant bits together, the FP32 exponent range), stored in the order (x1, x0, x2) so that
// both (x1, x0) and (x0, x2) are contiguous.  A product needs the partial products x_i * y_j with
// i + j <= 2 (the others are below 2^-24 relative).  tcgen05.mma takes as long for M = 128 as for
// M = 64 and only 1.4x as long for N = 128 as for N = 64, so the terms are stacked along both
// dimensions and a product is two MMAs per 16-wide K step instead of six:
//     [x1; x0] * [y1 | y0]  -> accumulator columns   0..127   (x1y1, x1y0 | x0y1, x0y0)
//     [x0; x2] * [y0 | y2]  -> accumulator columns 128..255   (x0y0*, x0y2 | x2y0, x2y2*)
// (* not used).  Rows 0..63 of the stacked left operand land in TMEM lanes 0..63, rows 64..127 in
// lanes 64..127, so the epilogue adds the wanted 64-column blocks inside each lane and then the
// two lane halves through a small shared-memory exchange between partner warps.  The tiles use
// the 128-byte swizzle ([64 rows x 128 B]); a matrix stored row-major serves as either operand,
// plain or transposed, by choosing the K-major or the MN-major shared-memory descriptor, so no
// transposed copies exist.  One CTA per (b,h) slice: 8 compute warps (256 threads) and a ninth
// warp whose first lane issues the MMAs.  After the exchange every compute thread owns 16
// consecutive columns of one row, applies the step's affine map and writes the next operand
// tiles; when its tiles are written it arrives on a "ready" mbarrier the issuing thread waits on.
// Independent products of a step are issued together with two commits, so the epilogue of the
// first group overlaps the MMAs of the second.  A wait that gives up (bounded, 1.5 s) marks the
// call failed in the status word; control flow never depends on it, so no barrier is missed.
// The set-up and the tail of the algorithm (softmax, ridge, norms, Z0 and its gradient) are the
// FP32 CUDA-core code of ns_kernels.cuh, run on FP32 staging buffers that alias the tile slots.
#pragma once
#include "ns_kernels.cuh"
#include "small_kernels.cuh"
#include "tc_common.cuh"

namespace fnb {
namespace nstc {

using namespace tc;
using ns::kBuf;
using ns::kLd;
using ns::kN;
using ns::Norms;

constexpr int kTileBytes = kN * 128;        // one bf16 term of a matrix
constexpr int kSet = 3 * kTileBytes;        // the three terms of a matrix, order (x1, x0, x2)
constexpr int kTerm0 = kTileBytes, kTerm1 = 0, kTerm2 = 2 * kTileBytes;
constexpr int kXchBytes = kN * kLd * 4;     // FP32 exchange buffer between the lane halves
constexpr int kFwdSlots = 7, kBwdSlots = 8;
constexpr size_t kFwdSmem = (size_t)kFwdSlots * kSet + kXchBytes + 1024;
constexpr size_t kBwdSmem = (size_t)kBwdSlots * kSet + kXchBytes + 1024;
constexpr uint32_t kFwdTmemCols = 256, kBwdTmemCols = 512;
constexpr uint32_t kAcc0 = 0, kAcc1 = 256;  // TMEM column of the two accumulators

// Optional phase timestamps of CTA 0 (profiling builds only).
#ifdef FNB_NS_TRACE
__device__ unsigned long long g_ns_span[2 * 64];   // per-CTA kernel entry / exit times
__device__ unsigned long long g_ns_trace[160];
__device__ int g_ns_trace_n;
#define NS_TRACE()                                                                                  \
  do {                                                                                              \
    if (blockIdx.x == 0 && threadIdx.x == 0 && g_ns_trace_n < 160) g_ns_trace[g_ns_trace_n++] = global_ns(); \
  } while (0)
#ifdef FNB_NS_TRACE_FINE
#define NS_TRACE2() NS_TRACE()
#else
#define NS_TRACE2() do {} while (0)
#endif
#else
#define NS_TRACE() do {} while (0)
#define NS_TRACE2() do {} while (0)
#endif

struct Ctx {
  uint8_t* base;        // 1024-byte aligned start of the tile slots
  float* xch;           // exchange buffer (row stride kLd)
  uint64_t* bar;        // two completion barriers (MMA groups -> compute warps)
  uint64_t* ready;      // operand tiles written (one arrival per compute warp -> issuing thread)
  uint32_t phase[2];    // parity the next wait on each completion barrier uses
  uint32_t rphase;      // parity the next wait on `ready` uses
  bool failed;          // a wait of this thread gave up
  uint32_t tmem;        // base address of the allocated tensor memory
  Abort ab;
  // epilogue role of this thread: TMEM lane 32*quarter + lane holds row `row` of the lane half
  // `part`; after the exchange the thread owns columns col0 .. col0+15 of that row
  int row, part, c32, col0, pair_bar;
  uint32_t lane_off;
  __device__ __forceinline__ uint8_t* slot(int i) const { return base + (size_t)i * kSet; }
  __device__ __forceinline__ uint32_t slot_addr(int i) const { return smem_u32(base) + (uint32_t)i * kSet; }
};

// ---- FP32 -> three bf16 terms ---------------------------------------------------------------
// 8 consecutive values of row r, columns 8*chunk .. 8*chunk+7 -> one 16-byte chunk per term
__device__ __forceinline__ void split_store8(uint8_t* set, int r, int chunk, const float* v) {
  uint32_t w0[4], w1[4], w2[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    float a = v[2 * p], b = v[2 * p + 1];
    w0[p] = pack2<__nv_bfloat16>(a, b);            // low half = a, high half = b
    a -= __uint_as_float(w0[p] << 16);
    b -= __uint_as_float(w0[p] & 0xffff0000u);
    w1[p] = pack2<__nv_bfloat16>(a, b);
    a -= __uint_as_float(w1[p] << 16);
    b -= __uint_as_float(w1[p] & 0xffff0000u);
    w2[p] = pack2<__nv_bfloat16>(a, b);
  }
  const uint32_t off = sw128_offset(r, chunk);
  *reinterpret_cast<uint4*>(set + kTerm0 + off) = make_uint4(w0[0], w0[1], w0[2], w0[3]);
  *reinterpret_cast<uint4*>(set + kTerm1 + off) = make_uint4(w1[0], w1[1], w1[2], w1[3]);
  *reinterpret_cast<uint4*>(set + kTerm2 + off) = make_uint4(w2[0], w2[1], w2[2], w2[3]);
}
// 16 values: columns col0 .. col0+15 of row r
__device__ __forceinline__ void split_store16(uint8_t* set, int r, int col0, const float* v) {
  split_store8(set, r, (col0 >> 3), v);
  split_store8(set, r, (col0 >> 3) + 1, v + 8);
}

// whole-matrix conversions: thread t handles row t >> 2, columns 16*(t & 3) .. +15
// dense global [rows x cols] matrix with row stride ld -> registers, zero beyond rows / cols
__device__ __forceinline__ void load_global16(const float* g, int rows, int cols, int ld, float* v) {
  const int r = threadIdx.x >> 2, c0 = (threadIdx.x & 3) * 16;
  if (((ld | cols) & 3) == 0) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int cc = c0 + 4 * q;
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < rows && cc < cols) x = *reinterpret_cast<const float4*>(g + (size_t)r * ld + cc);
      v[4 * q] = x.x; v[4 * q + 1] = x.y; v[4 * q + 2] = x.z; v[4 * q + 3] = x.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = (r < rows && c0 + i < cols) ? g[(size_t)r * ld + c0 + i] : 0.f;
  }
}
__device__ __forceinline__ void store_set16(uint8_t* set, const float* v) {
  split_store16(set, threadIdx.x >> 2, (threadIdx.x & 3) * 16, v);
}
__device__ __forceinline__ void store_buf16(float* X, const float* v) {
  float* dst = X + (threadIdx.x >> 2) * kLd + (threadIdx.x & 3) * 16;
#pragma unroll
  for (int q = 0; q < 4; ++q)
    *reinterpret_cast<float4*>(dst + 4 * q) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
}
// padded FP32 shared buffer (row stride kLd) -> tile set
__device__ __forceinline__ void convert_buf(uint8_t* set, const float* X) {
  const int r = threadIdx.x >> 2, c0 = (threadIdx.x & 3) * 16;
  float v[16];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float4 x = *reinterpret_cast<const float4*>(X + r * kLd + c0 + 4 * q);
    v[4 * q] = x.x; v[4 * q + 1] = x.y; v[4 * q + 2] = x.z; v[4 * q + 3] = x.w;
  }
  split_store16(set, r, c0, v);
}

// ---- products -------------------------------------------------------------------------------
// An operand is a tile set plus how the product reads it:
//   left operand  X (M x K):  plain = K-major,  transposed (X^T as left operand) = MN-major
//   right operand Y (K x N):  plain = MN-major, transposed (Y^T as right operand) = K-major
struct Operand { uint32_t addr; bool mn; };
__device__ __forceinline__ Operand left(uint32_t set) { return {set, false}; }
__device__ __forceinline__ Operand left_t(uint32_t set) { return {set, true}; }
__device__ __forceinline__ Operand right(uint32_t set) { return {set, true}; }
__device__ __forceinline__ Operand right_t(uint32_t set) { return {set, false}; }

// descriptor of two stacked term tiles starting `first` bytes into the set, K step k
__device__ __forceinline__ uint64_t pair_desc(const Operand& o, int first, int k) {
  const uint32_t tile = o.addr + (uint32_t)first;
  return o.mn ? smem_desc_sw128(tile + k * 2048, kTileBytes, 1024)   // 16 rows of K per step; the second
                                                                     // 64-wide block is the next tile
              : smem_desc_sw128(tile + k * 32, 16, 1024);            // 32 bytes of K per step; rows 64..127
                                                                     // continue into the next tile
}
// accumulator at TMEM address d (256 columns) (+)= a * b
__device__ __forceinline__ void issue_product(uint32_t d, Operand a, Operand b, bool accumulate) {
  const uint32_t idesc = make_idesc<__nv_bfloat16>(128, 128, a.mn, b.mn);
  uint32_t acc = accumulate ? 1u : 0u;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    umma(d, pair_desc(a, 0, k), pair_desc(b, 0, k), idesc, acc);                          // [x1;x0] [y1|y0]
    umma(d + 128, pair_desc(a, kTileBytes, k), pair_desc(b, kTileBytes, k), idesc, acc);  // [x0;x2] [y0|y2]
    acc = 1u;
  }
}

constexpr int kComputeThreads = 256;
constexpr int kNsTcThreads = kComputeThreads + 32;
__device__ __forceinline__ bool is_compute() { return threadIdx.x < kComputeThreads; }
__device__ __forceinline__ bool is_issuer() { return threadIdx.x == kComputeThreads; }

// compute side: my operand tiles (and my reads of the accumulators) are done
__device__ __forceinline__ void tiles_ready(Ctx& c) {
  fence_proxy_async();
  tc_fence_before();
  mbar_arrive_warp(c.ready);
}
// compute side: wait for MMA group g (0 or 1) of the current batch
__device__ __forceinline__ void wait_group(Ctx& c, int g, int where) {
  NS_TRACE2();
  if (!mbar_wait(c.bar + g, c.phase[g], c.ab, where)) c.failed = true;
  c.phase[g] ^= 1u;
  tc_fence_after();
  NS_TRACE2();
}
// issuing thread: wait for the operands, issue two groups of products, one commit each
template <class IssueA, class IssueB>
__device__ __forceinline__ void mma_batch(Ctx& c, int where, IssueA issue_a, IssueB issue_b) {
  if (!c.failed && !mbar_wait(c.ready, c.rphase, c.ab, where)) c.failed = true;
  c.rphase ^= 1u;
  if (c.failed) return;
  tc_fence_after();
  issue_a();
  umma_commit(c.bar);
  issue_b();
  umma_commit(c.bar + 1);
}
template <class Issue>
__device__ __forceinline__ void mma_single(Ctx& c, int where, Issue issue) {
  if (!c.failed && !mbar_wait(c.ready, c.rphase, c.ab, where)) c.failed = true;
  c.rphase ^= 1u;
  if (c.failed) return;
  tc_fence_after();
  issue();
  umma_commit(c.bar);
}

// Result of the accumulator at TMEM column `col`: after the call v[0..15] holds columns
// c.col0 .. c.col0+15 of row c.row.  Every thread must call (warp-wide TMEM loads, pair barriers).
__device__ __forceinline__ void acc_result(const Ctx& c, uint32_t col, float* v) {
  float s[32], t[32];
  const uint32_t a = c.tmem + col + c.lane_off;
  tmem_ld32(a, s);                          // lanes 0..63: x1y1 ; lanes 64..127: x0y1
  tmem_ld32(a + 64, t);                     //              x1y0 ;                x0y0
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) s[i] += t[i];
  NS_TRACE2();
  tmem_ld32(a + (c.part ? 128 : 192), t);   //              x0y2 ;                x2y0
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) s[i] += t[i];
  NS_TRACE2();
  // hand the 16 columns the partner finalises over, take the partner's share of mine
  // (part is warp-uniform; the two branches keep every register index a constant)
  float* rowp = c.xch + c.row * kLd + c.c32;
  if (c.part == 0) {
#pragma unroll
    for (int q = 0; q < 4; ++q)
      *reinterpret_cast<float4*>(rowp + 16 + 4 * q) = make_float4(s[16 + 4 * q], s[17 + 4 * q], s[18 + 4 * q], s[19 + 4 * q]);
    named_barrier(c.pair_bar, 64);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4 x = *reinterpret_cast<const float4*>(rowp + 4 * q);
      v[4 * q] = s[4 * q] + x.x; v[4 * q + 1] = s[4 * q + 1] + x.y;
      v[4 * q + 2] = s[4 * q + 2] + x.z; v[4 * q + 3] = s[4 * q + 3] + x.w;
    }
  } else {
#pragma unroll
    for (int q = 0; q < 4; ++q)
      *reinterpret_cast<float4*>(rowp + 4 * q) = make_float4(s[4 * q], s[4 * q + 1], s[4 * q + 2], s[4 * q + 3]);
    named_barrier(c.pair_bar, 64);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4 x = *reinterpret_cast<const float4*>(rowp + 16 + 4 * q);
      v[4 * q] = s[16 + 4 * q] + x.x; v[4 * q + 1] = s[17 + 4 * q] + x.y;
      v[4 * q + 2] = s[18 + 4 * q] + x.z; v[4 * q + 3] = s[19 + 4 * q] + x.w;
    }
  }
  named_barrier(c.pair_bar, 64);   // the partner has read: the exchange buffer may be reused
  NS_TRACE2();
}

// v[i] = s * v[i] + (diagonal ? d : 0), diagonal restricted to the leading m x m block
__device__ __forceinline__ void affine(const Ctx& c, float* v, float s, float d, int m) {
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = s * v[i] + ((c.col0 + i == c.row && c.row < m) ? d : 0.f);
}
// this thread's row segment, restricted to the leading rows x cols block -> dense global matrix
__device__ __forceinline__ void store_global16(const Ctx& c, float* g, const float* v, int rows, int cols, int ld) {
  if (c.row >= rows) return;
  if (((ld | cols) & 3) == 0) {
#pragma unroll
    for (int i = 0; i < 16; i += 4)
      if (c.col0 + i < cols)
        *reinterpret_cast<float4*>(g + (size_t)c.row * ld + c.col0 + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (c.col0 + i < cols) g[(size_t)c.row * ld + c.col0 + i] = v[i];
  }
}
__device__ __forceinline__ void store_row16(const Ctx& c, float* X, const float* v) {
#pragma unroll
  for (int i = 0; i < 16; i += 4)
    *reinterpret_cast<float4*>(X + c.row * kLd + c.col0 + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
}

// common set-up / teardown of the kernels below (called by all 288 threads)
struct Shared {
  uint64_t bar[2];
  uint64_t ready;
  uint32_t tmem_slot;
  int abort_word;
};
__device__ __forceinline__ void ctx_open(Ctx& c, Shared& sh, uint8_t* dyn, int slots, int* status, uint32_t cols) {
  c.base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn) + 1023) & ~(uintptr_t)1023);
  c.xch = reinterpret_cast<float*>(c.base + (size_t)slots * kSet);
  c.bar = sh.bar;
  c.ready = &sh.ready;
  c.phase[0] = c.phase[1] = c.rphase = 0;
  c.failed = false;
  c.ab.flag = &sh.abort_word;
  c.ab.status = status;
  const int warp = (threadIdx.x >> 5) & 7, lane = threadIdx.x & 31, quarter = warp & 3, half = warp >> 2;
  c.part = quarter >> 1;
  c.row = (quarter & 1) * 32 + lane;
  c.c32 = half * 32;
  c.col0 = c.c32 + 16 * c.part;
  c.pair_bar = 1 + (quarter & 1) + 2 * half;      // warps w and w ^ 2 share a barrier
  c.lane_off = ((uint32_t)(quarter * 32) << 16) + (uint32_t)c.c32;
  if (threadIdx.x == 0) {
    sh.abort_word = 0;
    mbar_init(&sh.bar[0], 1);
    mbar_init(&sh.bar[1], 1);
    mbar_init(&sh.ready, kComputeThreads / 32);
    fence_mbar_init();
  }
  if (threadIdx.x < 32) {
    tmem_alloc(&sh.tmem_slot, cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  c.tmem = sh.tmem_slot;
}
__device__ __forceinline__ void ctx_close(Ctx& c, uint32_t cols) {
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) tmem_dealloc(c.tmem, cols);
}

// ---------------------------------------------------------------------------------------------
// Forward.  Slots: 0 A, 1 Z, 2 M, 3 nU = M - 7I, 4 V, 5 qT = T / 4, 6 K2 (ridge only).
// FP32 staging (K2, A) aliases slots 2..4; in: K2 (softmaxed, padded) in staging buffer 0.
__device__ __forceinline__ float* fwd_staging(const Ctx& c) { return reinterpret_cast<float*>(c.slot(2)); }

// issuing thread: the products of the forward in the order the compute warps consume them
__device__ inline void pinv_forward_issue(Ctx& c, int J, float kappa, bool scores) {
  const uint32_t sA = c.slot_addr(0), sZ = c.slot_addr(1), sM = c.slot_addr(2), sU = c.slot_addr(3),
                 sV = c.slot_addr(4), sT = c.slot_addr(5), sK2 = c.slot_addr(6);
  const uint32_t acc0 = c.tmem + kAcc0;
  if (scores) mma_single(c, 0x20ff, [&] { issue_product(acc0, left(sA), right_t(sZ), false); });   // Qt Kt^T
  for (int j = 0; j < J; ++j) {
    mma_single(c, 0x2100, [&] { issue_product(acc0, left(sA), right(sZ), false); });
    mma_single(c, 0x2101, [&] { issue_product(acc0, left(sM), right(sU), false); });
    mma_single(c, 0x2102, [&] { issue_product(acc0, left(sM), right(sV), false); });
    mma_single(c, 0x2103, [&] { issue_product(acc0, left(sZ), right(sT), false); });
  }
  if (kappa > 0.f) mma_single(c, 0x2104, [&] { issue_product(acc0, left(sZ), right_t(sK2), false); });
}

// compute warps
__device__ inline void pinv_forward_tc(Ctx& c, float* red, float* iterates, float* k2inv, int m, int J,
                                       float kappa) {
  float* bK2 = fwd_staging(c);
  float* bA = bK2 + kBuf;
  const int mm_ = m * m;
  const float* A = bK2;
  if (kappa > 0.f) {
    Norms nk = ns::norms(bK2, m, red);
    const float lam = nk.n1 * nk.ninf / kappa;
    ns::mm<ns::TN>(bK2, bK2, [&](int r, int cc, float acc) { bA[r * kLd + cc] = acc + ((r == cc && r < m) ? lam : 0.f); });
    A = bA;
    convert_buf(c.slot(6), bK2);
  }
  Norms na = ns::norms(A, m, red);
  const float cden = fmaxf(na.n1 * na.ninf, 1e-12f);
  {
    // Z0 = A^T / cden -> slot 1 and iterates[0] (and the result itself when there is no iteration)
    const int r = threadIdx.x >> 2, c0 = (threadIdx.x & 3) * 16;
    float z[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) z[i] = A[(c0 + i) * kLd + r] / cden;
    split_store16(c.slot(1), r, c0, z);
    if (r < m) {
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (c0 + i < m) {
          iterates[r * m + c0 + i] = z[i];
          if (J == 0 && !(kappa > 0.f)) k2inv[r * m + c0 + i] = z[i];
        }
    }
  }
  convert_buf(c.slot(0), A);
  NS_TRACE();
  float v[16];
  for (int j = 0; j < J; ++j) {
    float* Zn = iterates + (size_t)(j + 1) * mm_;
    NS_TRACE();
    tiles_ready(c);
    wait_group(c, 0, 0x2110);
    acc_result(c, kAcc0, v);
    split_store16(c.slot(2), c.row, c.col0, v);
    affine(c, v, 1.f, -7.f, m);
    split_store16(c.slot(3), c.row, c.col0, v);
    tiles_ready(c);
    wait_group(c, 0, 0x2111);
    acc_result(c, kAcc0, v);
    affine(c, v, 1.f, 15.f, m);
    split_store16(c.slot(4), c.row, c.col0, v);
    tiles_ready(c);
    wait_group(c, 0, 0x2112);
    acc_result(c, kAcc0, v);
    affine(c, v, -0.25f, 3.25f, m);
    split_store16(c.slot(5), c.row, c.col0, v);
    tiles_ready(c);
    wait_group(c, 0, 0x2113);
    acc_result(c, kAcc0, v);
    split_store16(c.slot(1), c.row, c.col0, v);
    if (!c.failed) {
      store_global16(c, Zn, v, m, m, m);
      if (j == J - 1 && !(kappa > 0.f)) store_global16(c, k2inv, v, m, m, m);
    }
  }
  NS_TRACE();
  if (kappa > 0.f) {
    // k2inv = Z_J K2^T
    tiles_ready(c);
    wait_group(c, 0, 0x2114);
    acc_result(c, kAcc0, v);
    if (!c.failed) store_global16(c, k2inv, v, m, m, m);
  }
}

// Scores S2 = Qt Kt^T for head_dim 64 as one split product (Qt in slot 0, Kt in slot 1, both
// overwritten afterwards), then the FP32 row softmax.
__device__ inline void s2_softmax_tc(Ctx& c, const ns::NsFwdParams& p, int64_t bh) {
  const int m = p.m, D = p.D;
  float q[16], k[16], v[16];
  if (p.land) {
    pooled_row16(p.land, 0, p.BH, bh, m, p.C, p.seg_N, p.scale, q);
    pooled_row16(p.land, 1, p.BH, bh, m, p.C, p.seg_N, p.scale, k);
    const int r = threadIdx.x >> 2, c0 = (threadIdx.x & 3) * 16;
    if (r < m) {
      float4* dq = reinterpret_cast<float4*>(p.qt_out + (bh * m + r) * D + c0);
      float4* dk = reinterpret_cast<float4*>(p.kt_out + (bh * m + r) * D + c0);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        dq[i] = make_float4(q[4 * i], q[4 * i + 1], q[4 * i + 2], q[4 * i + 3]);
        dk[i] = make_float4(k[4 * i], k[4 * i + 1], k[4 * i + 2], k[4 * i + 3]);
      }
    }
  } else {
    load_global16(p.qt + bh * m * D, m, D, D, q);
    load_global16(p.kt + bh * m * D, m, D, D, k);
  }
  store_set16(c.slot(0), q);
  store_set16(c.slot(1), k);
  tiles_ready(c);
  wait_group(c, 0, 0x210f);
  acc_result(c, kAcc0, v);
  store_row16(c, fwd_staging(c), v);
  ns::ns_sync();
  ns::softmax_rows(fwd_staging(c), p, bh);
}

__global__ void __launch_bounds__(kNsTcThreads, 1) ns_fwd_tc_kernel(ns::NsFwdParams p, int* status) {
  extern __shared__ uint8_t dyn_smem[];
  __shared__ float red[ns::kRedFloats];
  __shared__ Shared sh;
  Ctx c;
  ctx_open(c, sh, dyn_smem, kFwdSlots, status, kFwdTmemCols);
  const int64_t bh = blockIdx.x;
  const int m = p.m;
  const bool scores_tc = p.D == kN;
  if (is_compute()) {
    NS_TRACE();
    if (scores_tc) s2_softmax_tc(c, p, bh);
    else ns::s2_softmax(fwd_staging(c), p, bh);
    NS_TRACE();
    pinv_forward_tc(c, red, p.iterates + bh * (size_t)(p.J + 1) * m * m, p.k2inv + bh * m * m, m, p.J, p.kappa);
  } else if (is_issuer()) {
    pinv_forward_issue(c, p.J, p.kappa, scores_tc);
  }
  ctx_close(c, kFwdTmemCols);
}

__global__ void __launch_bounds__(kNsTcThreads, 1)
ns_pinv_fwd_tc_debug_kernel(const float* k2, float* iterates, float* k2inv, int m, int J, float kappa,
                            int* status) {
  extern __shared__ uint8_t dyn_smem[];
  __shared__ float red[ns::kRedFloats];
  __shared__ Shared sh;
  Ctx c;
  ctx_open(c, sh, dyn_smem, kFwdSlots, status, kFwdTmemCols);
  const int64_t bh = blockIdx.x;
  if (is_compute()) {
    ns::load_mat(fwd_staging(c), k2 + bh * m * m, m);
    ns::ns_sync();
    pinv_forward_tc(c, red, iterates + bh * (size_t)(J + 1) * m * m, k2inv + bh * m * m, m, J, kappa);
  } else if (is_issuer()) {
    pinv_forward_issue(c, J, kappa, false);
  }
  ctx_close(c, kFwdTmemCols);
}

// ---------------------------------------------------------------------------------------------
// Backward.  Slots: 0 A, 1 Z_j, 2 dZ (gradient w.r.t. Z_{j+1}), 3 M, 4 nU = M - 7I,
// 5 ndT = -dT, 6 V then qT = T / 4, 7 dV then dM.  Two TMEM accumulators.  Per iteration, with
// dT = Z^T dZ / 4, dV = -M^T dT, dU = -M^T dV:
//   batch 1:  M = A Z                         | ndT = -(Z^T dZ) / 4
//   batch 2:  V = 15 I + M nU                 | dV  = M^T ndT
//   batch 3:  dM = ndT V^T + dV nU^T + M^T dV | qT = (13 I - M V) / 4
//   batch 4:  dZ' = dZ qT^T + A^T dM          | dA += dM Z^T   (dA lives in registers)
// The epilogue of the group left of the bar runs while the group right of it is still in the
// tensor core.  The next iterate is fetched into registers a whole iteration ahead.  With the
// ridge the FP32 set-up (K2, A, Z_J, dZ_J) is staged in slots 5..7; after the loop the tail
// works in FP32 buffers at the start of the slot area.  A last batch (head_dim 64 only) forms the
// landmark gradients dqt_ns = dS2 Kt and dS2^T Qt from slots 5 (dS2), 6 (Kt), 7 (Qt); head_dim 128
// runs it twice, once per 64 columns of Kt and Qt.
constexpr int kBwdStageSlot = 5;
__device__ __forceinline__ float* bwd_stage(const Ctx& c, int i) {
  return reinterpret_cast<float*>(c.slot(kBwdStageSlot)) + (size_t)i * kBuf;
}
__device__ __forceinline__ float* bwd_tail(const Ctx& c, int i) {
  return reinterpret_cast<float*>(c.base) + (size_t)i * kBuf;
}

// issuing thread
__device__ inline void pinv_backward_issue(Ctx& c, int J, int finish, bool head) {
  if (head) {
    // dO3 = K2inv^T dstep2 | dK2inv = dstep2 Bmat^T   (slots 3 K2inv, 4 dstep2, 6 Bmat)
    const uint32_t sKi = c.slot_addr(3), sDs = c.slot_addr(4), sBm = c.slot_addr(6);
    mma_batch(c, 0x21f0, [&] { issue_product(c.tmem + kAcc0, left_t(sKi), right(sDs), false); },
              [&] { issue_product(c.tmem + kAcc1, left(sDs), right_t(sBm), false); });
  }
  const uint32_t sA = c.slot_addr(0), sZ = c.slot_addr(1), sdZ = c.slot_addr(2), sM = c.slot_addr(3),
                 sU = c.slot_addr(4), sdT = c.slot_addr(5), sV = c.slot_addr(6), sT = c.slot_addr(6),
                 sdV = c.slot_addr(7), sdM = c.slot_addr(7);
  const uint32_t acc0 = c.tmem + kAcc0, acc1 = c.tmem + kAcc1;
  for (int j = J - 1; j >= 0; --j) {
    mma_batch(c, 0x2200, [&] { issue_product(acc0, left(sA), right(sZ), false); },
              [&] { issue_product(acc1, left_t(sZ), right(sdZ), false); });
    mma_batch(c, 0x2201, [&] { issue_product(acc0, left(sM), right(sU), false); },
              [&] { issue_product(acc1, left_t(sM), right(sdT), false); });
    mma_batch(c, 0x2202,
              [&] {
                issue_product(acc1, left(sdT), right_t(sV), false);
                issue_product(acc1, left(sdV), right_t(sU), true);
                issue_product(acc1, left_t(sM), right(sdV), true);
              },
              [&] { issue_product(acc0, left(sM), right(sV), false); });
    mma_batch(c, 0x2203,
              [&] {
                issue_product(acc0, left(sdZ), right_t(sT), false);
                issue_product(acc0, left_t(sA), right(sdM), true);
              },
              [&] { issue_product(acc1, left(sdM), right_t(sZ), false); });
  }
  for (int half = 0; half < finish; ++half) {
    const uint32_t sS = c.slot_addr(5), sK = c.slot_addr(6), sQ = c.slot_addr(7);
    mma_batch(c, 0x2204, [&] { issue_product(acc0, left(sS), right(sK), false); },
              [&] { issue_product(acc1, left_t(sS), right(sQ), false); });
  }
}

// compute warps.  Requires J >= 1.  Returns dK2 (padded FP32 buffer); K2 is left in bwd_tail(c, 0).
// before_tail() runs between the iterations and the FP32 tail (a place to start global loads
// whose latency the tail hides).
template <class BeforeTail>
__device__ __forceinline__ float* pinv_backward_tc(Ctx& c, float* red, const float* k2g, const float* iterates,
                                                   const float* G, float* spill, int m, int J, float kappa,
                                                   BeforeTail before_tail, float* step_dz = nullptr,
                                                   float* step_da = nullptr) {
  // G == nullptr: dL/dk2inv is already in place (slot 2 without the ridge, staging buffer 3 with it)
  const int mm_ = m * m;
  float znext[16];
  load_global16(iterates + (size_t)(J - 1) * mm_, m, m, m, znext);
  if (kappa > 0.f) {
    float* bK2 = bwd_stage(c, 0);
    float* bA = bwd_stage(c, 1);
    float* bZ = bwd_stage(c, 2);
    float* bdZ = bwd_stage(c, 3);
    ns::load_mat(bK2, k2g, m);
    if (G) ns::load_mat(bdZ, G, m);
    ns::ns_sync();
    Norms nk = ns::norms(bK2, m, red);
    const float lam = nk.n1 * nk.ninf / kappa;
    ns::mm<ns::TN>(bK2, bK2, [&](int r, int cc, float acc) { bA[r * kLd + cc] = acc + ((r == cc && r < m) ? lam : 0.f); });
    ns::load_mat(bZ, iterates + (size_t)J * mm_, m);
    ns::ns_sync();
    // dK2_a = G^T Z_J -> global spill; dZ_J = G K2
    ns::mm<ns::TN>(bdZ, bZ, [&](int r, int cc, float acc) { if (r < m && cc < m) spill[r * m + cc] = acc; });
    ns::mm<ns::NN>(bdZ, bK2, [&](int r, int cc, float acc) { bdZ[r * kLd + cc] = acc; });
    convert_buf(c.slot(0), bA);
    convert_buf(c.slot(2), bdZ);
  } else {
    // A = K2 and dZ_J = G go straight from global memory into their tiles
    float a[16];
    load_global16(k2g, m, m, m, a);
    if (G) {
      float g[16];
      load_global16(G, m, m, m, g);
      store_set16(c.slot(2), g);
    }
    store_set16(c.slot(0), a);
  }
  store_set16(c.slot(1), znext);
  NS_TRACE();
  float v[16], dA[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) dA[i] = 0.f;
  for (int j = J - 1; j >= 0; --j) {
    tiles_ready(c);
    // next iterate; in the last iteration K2 for the FP32 tail instead
    load_global16(j > 0 ? iterates + (size_t)(j - 1) * mm_ : k2g, m, m, m, znext);
    wait_group(c, 0, 0x2210);
    acc_result(c, kAcc0, v);
    split_store16(c.slot(3), c.row, c.col0, v);
    affine(c, v, 1.f, -7.f, m);
    split_store16(c.slot(4), c.row, c.col0, v);
    wait_group(c, 1, 0x2220);
    acc_result(c, kAcc1, v);
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] *= -0.25f;
    split_store16(c.slot(5), c.row, c.col0, v);
    NS_TRACE();
    tiles_ready(c);
    wait_group(c, 0, 0x2211);
    acc_result(c, kAcc0, v);
    affine(c, v, 1.f, 15.f, m);
    split_store16(c.slot(6), c.row, c.col0, v);
    wait_group(c, 1, 0x2221);
    acc_result(c, kAcc1, v);
    split_store16(c.slot(7), c.row, c.col0, v);
    NS_TRACE();
    tiles_ready(c);
    wait_group(c, 0, 0x2212);
    acc_result(c, kAcc1, v);
    split_store16(c.slot(7), c.row, c.col0, v);      // dM over dV: every product reading dV is done
    wait_group(c, 1, 0x2222);
    acc_result(c, kAcc0, v);
    affine(c, v, -0.25f, 3.25f, m);
    split_store16(c.slot(6), c.row, c.col0, v);      // qT over V
    NS_TRACE();
    tiles_ready(c);
    wait_group(c, 0, 0x2213);
    acc_result(c, kAcc0, v);
    if (j > 0) split_store16(c.slot(2), c.row, c.col0, v);
    wait_group(c, 1, 0x2223);
    // every product of this iteration is complete: all tiles are free
    if (j == 0) store_row16(c, bwd_tail(c, 2), v);
    acc_result(c, kAcc1, v);
#pragma unroll
    for (int i = 0; i < 16; ++i) dA[i] += v[i];
    if (j > 0) store_set16(c.slot(1), znext);
    NS_TRACE();
  }
  if (step_dz) {
    // isolation hook: hand back dL/dZ_0 and the dL/dA accumulated over the iterations, skip the tail
    ns::ns_sync();
    if (!c.failed) {
      ns::store_mat(step_dz, bwd_tail(c, 2), m);
      store_global16(c, step_da, dA, m, m, m);
    }
    return nullptr;
  }
  before_tail();
  store_row16(c, bwd_tail(c, 3), dA);
  float* bK2 = bwd_tail(c, 0);
  float* bA = bwd_tail(c, 1);
  store_buf16(bK2, znext);
  ns::ns_sync();
  NS_TRACE();
  const float* A = bK2;
  if (kappa > 0.f) {
    Norms nk = ns::norms(bK2, m, red);
    const float lam = nk.n1 * nk.ninf / kappa;
    ns::mm<ns::TN>(bK2, bK2, [&](int r, int cc, float acc) { bA[r * kLd + cc] = acc + ((r == cc && r < m) ? lam : 0.f); });
    A = bA;
  }
  return ns::pinv_backward_tail(bK2, A, bwd_tail(c, 2), bwd_tail(c, 3), bwd_tail(c, 4), bwd_tail(c, 5), red, spill,
                                m, kappa);
}

__global__ void __launch_bounds__(kNsTcThreads, 1)
ns_pinv_bwd_tc_debug_kernel(const float* k2, const float* iterates, const float* G, float* dK2, float* spill,
                            int m, int J, float kappa, int* status, float* step_dz, float* step_da) {
  extern __shared__ uint8_t dyn_smem[];
  __shared__ float red[ns::kRedFloats];
  __shared__ Shared sh;
  Ctx c;
  ctx_open(c, sh, dyn_smem, kBwdSlots, status, kBwdTmemCols);
  const int64_t bh = blockIdx.x;
  if (is_compute()) {
    // step hook: one iteration (J = 1) whose "iterates" is the single matrix Z_j per slice
    const float* its = step_dz ? iterates + bh * (size_t)m * m : iterates + bh * (size_t)(J + 1) * m * m;
    float* out = pinv_backward_tc(c, red, k2 + bh * m * m, its, G + bh * m * m, spill + bh * m * m, m, J, kappa, [] {},
                                  step_dz ? step_dz + bh * m * m : nullptr, step_da ? step_da + bh * m * m : nullptr);
    if (out && !c.failed) ns::store_mat(dK2 + bh * m * m, out, m);
  } else if (is_issuer()) {
    pinv_backward_issue(c, J, false, false);
  }
  ctx_close(c, kBwdTmemCols);
}

// Softmax-2 Jacobian and the landmark gradients after the pseudoinverse backward, for head_dim 64
// and 128: dqt_ns = dS2 Kt and dkt_tot = dkt_a + dS2^T Qt as one more batch of split products per
// 64 columns of the landmarks.
// bK2, dK2: padded FP32 buffers inside the tail area (slots 0..4); slots 5..7 take the operands.
struct FinishOperands { float kt[16], qt[16], da[16]; };
// global loads of the finishing step for columns [64 half, 64 half + 64); the first half is issued
// early so that its latency hides behind the tail
__device__ __forceinline__ void finish_load(const Ctx& c, const ns::NsBwdParams& p, int64_t bh, int half,
                                            FinishOperands& f) {
  const int m = p.m, D = p.D, md = m * D;
  load_global16(p.kt + bh * md + half * kN, m, kN, D, f.kt);
  load_global16(p.qt + bh * md + half * kN, m, kN, D, f.qt);
  // dkt_a for the row segment this thread finalises
  const float* src = p.dkt_a + bh * md + (size_t)c.row * D + half * kN + c.col0;
#pragma unroll
  for (int i = 0; i < 16; i += 4) {
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c.row < m) x = *reinterpret_cast<const float4*>(src + i);
    f.da[i] = x.x; f.da[i + 1] = x.y; f.da[i + 2] = x.z; f.da[i + 3] = x.w;
  }
}
template <int NH>
__device__ inline void ns_bwd_finish_tc(Ctx& c, const ns::NsBwdParams& p, int64_t bh, const float* bK2, float* dK2,
                                        FinishOperands& f) {
  const int m = p.m, D = p.D, md = m * D, t = threadIdx.x;
  // softmax-2 Jacobian in place: dS2 = K2 o (dK2 - rowsum(dK2 o K2))
  const int w = t >> 5, lane = t & 31;
  for (int r = w; r < kN; r += kComputeThreads / 32) {
    float a0 = dK2[r * kLd + lane], a1 = dK2[r * kLd + lane + 32];
    float k0 = bK2[r * kLd + lane], k1 = bK2[r * kLd + lane + 32];
    float s = a0 * k0 + a1 * k1;
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    dK2[r * kLd + lane] = k0 * (a0 - s);
    dK2[r * kLd + lane + 32] = k1 * (a1 - s);
  }
  ns::ns_sync();
  convert_buf(c.slot(5), dK2);
#pragma unroll
  for (int half = 0; half < NH; ++half) {
    // every product that read slots 6 and 7 has been waited for below
    if (half > 0) finish_load(c, p, bh, half, f);
    store_set16(c.slot(6), f.kt);
    store_set16(c.slot(7), f.qt);
    tiles_ready(c);
    const size_t off = (size_t)bh * md + half * kN;
    float v[16];
    wait_group(c, 0, 0x2214);
    acc_result(c, kAcc0, v);
    if (!c.failed) store_global16(c, p.dqt_ns + off, v, m, kN, D);
    wait_group(c, 1, 0x2224);
    acc_result(c, kAcc1, v);
    if (c.failed) return;
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] += f.da[i];
    store_global16(c, p.dkt_tot + off, v, m, kN, D);
    if (p.rows_k && c.row < m) {
      Segments sg(p.N, m);
      const float fk = p.scale / (float)sg.len(c.row);
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] *= fk;
      store_global16(c, p.rows_k + off, v, m, kN, D);
    }
  }
}

// Head of the fused backward middle stage (head_dim 64): reduce the per-CTA partials of the
// softmax-1 pass, then dO3 = K2inv^T dstep2 (-> D3, normalised 16-bit copy for the column pass) and
// dK2inv = dstep2 Bmat^T, which lands where the pseudoinverse backward expects dL/dk2inv.
struct BwdHeadParams {
  const float* partA;         // [BH][nchunk][2][m][D]: dstep2 partials, dKt partials
  int nchunk;
  const float* k2inv; const float* bmat;
  float* dkt_a;               // [BH][m][D] out
  // The four outputs below feed the column pass; all are skipped when D3 is null (the column pass
  // then runs beside this kernel and takes them from a separate small kernel).
  float* D3;                  // [BH][m] out
  void* do3n;                 // [BH][MP][D] 16-bit out = dO3 / do3_scale
  float* do3_scale;           // [BH] out
  void* qt16;                 // [BH][MP][D] 16-bit out = qt_mul * Qt
  float qt_mul;
  int dtype, MP;
};

__device__ inline void bwd_head_tc(Ctx& c, float* red, const ns::NsBwdParams& p, const BwdHeadParams& h, int64_t bh) {
  const int m = p.m, D = p.D, md = m * D, t = threadIdx.x;
  const int r = t >> 2, c0 = (t & 3) * 16;
  NS_TRACE();
  // reduce the partials: this thread owns row r, columns c0 .. c0+15 of both sums
  float ds[16], dk[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) { ds[i] = 0.f; dk[i] = 0.f; }
  if (r < m) {
    const float* base = h.partA + bh * (int64_t)h.nchunk * 2 * md + (size_t)r * D + c0;
    constexpr int CB = 3;
    for (int ch0 = 0; ch0 < h.nchunk; ch0 += CB) {
      float4 x[CB][4], y[CB][4];
#pragma unroll
      for (int i = 0; i < CB; ++i) {
        const int ch = min(ch0 + i, h.nchunk - 1);
        const float4* s0 = reinterpret_cast<const float4*>(base + (size_t)ch * 2 * md);
        const float4* s1 = reinterpret_cast<const float4*>(base + (size_t)ch * 2 * md + md);
#pragma unroll
        for (int q = 0; q < 4; ++q) { x[i][q] = s0[q]; y[i][q] = s1[q]; }
      }
#pragma unroll
      for (int i = 0; i < CB; ++i)
        if (ch0 + i < h.nchunk) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            ds[4 * q] += x[i][q].x; ds[4 * q + 1] += x[i][q].y; ds[4 * q + 2] += x[i][q].z; ds[4 * q + 3] += x[i][q].w;
            dk[4 * q] += y[i][q].x; dk[4 * q + 1] += y[i][q].y; dk[4 * q + 2] += y[i][q].z; dk[4 * q + 3] += y[i][q].w;
          }
        }
    }
    float4* out = reinterpret_cast<float4*>(h.dkt_a + bh * md + (size_t)r * D + c0);
#pragma unroll
    for (int q = 0; q < 4; ++q) out[q] = make_float4(dk[4 * q], dk[4 * q + 1], dk[4 * q + 2], dk[4 * q + 3]);
  }
  NS_TRACE();
  store_set16(c.slot(4), ds);
  {
    float ki[16], bm[16];
    load_global16(h.k2inv + bh * m * m, m, m, m, ki);
    load_global16(h.bmat + bh * md, m, D, D, bm);
    store_set16(c.slot(3), ki);
    store_set16(c.slot(6), bm);
  }
  tiles_ready(c);
  NS_TRACE();
  // operands of this thread's share of the epilogue: Bmat segment for D3, Qt row for the copy
  float bseg[16], qrow[16];
  {
    const float* src = h.bmat + bh * md + (size_t)c.row * D + c.col0;
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c.row < m) x = *reinterpret_cast<const float4*>(src + i);
      bseg[i] = x.x; bseg[i + 1] = x.y; bseg[i + 2] = x.z; bseg[i + 3] = x.w;
    }
  }
  load_global16(p.qt + bh * md, m, D, D, qrow);
  float v[16];
  wait_group(c, 0, 0x21f1);
  acc_result(c, kAcc0, v);                       // dO3
  float d3 = 0.f, amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) { d3 = fmaf(v[i], bseg[i], d3); amax = fmaxf(amax, fabsf(v[i])); }
  float* do3f = bwd_tail(c, 0);                  // FP32 dO3 until the scale is known (slots 0, 1 are still free)
  store_row16(c, do3f, v);
  // red: [0..255] D3 partials (4 per row), [256..263] per-warp maxima
  red[c.row * 4 + (c.c32 >> 5) * 2 + c.part] = d3;
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((t & 31) == 0) red[256 + (t >> 5)] = amax;
  wait_group(c, 1, 0x21f2);
  acc_result(c, kAcc1, v);                       // dK2inv
  if (p.kappa > 0.f) store_row16(c, bwd_stage(c, 3), v);
  else split_store16(c.slot(2), c.row, c.col0, v);
  ns::ns_sync();
  float cmax = red[256];
#pragma unroll
  for (int w = 1; w < kComputeThreads / 32; ++w) cmax = fmaxf(cmax, red[256 + w]);
  const float sc = pow2_scale(cmax), inv_sc = 1.f / sc;
  if (h.D3) {
  if (t == 0) h.do3_scale[bh] = sc;
  if (t < m) h.D3[bh * m + t] = (red[4 * t] + red[4 * t + 1]) + (red[4 * t + 2] + red[4 * t + 3]);
  {
    // 16-bit copies, rows >= m zero: dO3 / scale and qt_mul * Qt
    const size_t ob = (size_t)bh * h.MP * D;
    uint32_t w0[8], w1[8];
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      const float a = (r < m) ? do3f[r * kLd + c0 + i] * inv_sc : 0.f;
      const float b = (r < m) ? do3f[r * kLd + c0 + i + 1] * inv_sc : 0.f;
      w0[i >> 1] = h.dtype == 1 ? pack2<__half>(a, b) : pack2<__nv_bfloat16>(a, b);
      w1[i >> 1] = h.dtype == 1 ? pack2<__half>(qrow[i] * h.qt_mul, qrow[i + 1] * h.qt_mul)
                                : pack2<__nv_bfloat16>(qrow[i] * h.qt_mul, qrow[i + 1] * h.qt_mul);
    }
    if (r < h.MP) {
      uint4* d0 = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(h.do3n) + ob + (size_t)r * D + c0);
      uint4* d1 = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(h.qt16) + ob + (size_t)r * D + c0);
      d0[0] = make_uint4(w0[0], w0[1], w0[2], w0[3]); d0[1] = make_uint4(w0[4], w0[5], w0[6], w0[7]);
      d1[0] = make_uint4(w1[0], w1[1], w1[2], w1[3]); d1[1] = make_uint4(w1[4], w1[5], w1[6], w1[7]);
    }
  }
  }
  ns::ns_sync();   // do3f (slots 0, 1) is free again
  NS_TRACE();
}

// NH: batches of the finishing step = head_dim / 64 for head_dim 64 and 128 (the instantiation with
// NH = 1 also serves the smaller head dims, whose finishing step runs on the CUDA cores)
template <int NH>
__global__ void __launch_bounds__(kNsTcThreads, 1)
ns_bwd_tc_kernel(ns::NsBwdParams p, BwdHeadParams h, int* status) {
  extern __shared__ uint8_t dyn_smem[];
#ifdef FNB_NS_TRACE
  if (threadIdx.x == 0 && blockIdx.x < 64) g_ns_span[2 * blockIdx.x] = global_ns();
#endif
  __shared__ float red[ns::kRedFloats];
  __shared__ Shared sh;
  Ctx c;
  NS_TRACE();
  pdl_trigger();
  ctx_open(c, sh, dyn_smem, kBwdSlots, status, kBwdTmemCols);
  pdl_wait();
  NS_TRACE();
  const int64_t bh = blockIdx.x;
  const int m = p.m, mm_ = m * m;
  const int finish_tc = p.D == NH * kN ? NH : 0;   // batches of the finishing step
  const bool head = h.partA != nullptr;      // fused middle stage (head_dim 64 only)
  if (is_compute()) {
    if (head) bwd_head_tc(c, red, p, h, bh);
    FinishOperands fo;
    float* dK2 = pinv_backward_tc(c, red, p.k2 + bh * mm_, p.iterates + bh * (size_t)(p.J + 1) * mm_,
                                  head ? nullptr : p.G + bh * mm_,
                                  p.spill + bh * mm_, m, p.J, p.kappa, [&] { if (finish_tc) finish_load(c, p, bh, 0, fo); });
    NS_TRACE();
    if (finish_tc) ns_bwd_finish_tc<NH>(c, p, bh, bwd_tail(c, 0), dK2, fo);
    else if (!c.failed) ns::ns_bwd_finish(p, bh, bwd_tail(c, 0), dK2);
    NS_TRACE();
  } else if (is_issuer()) {
    pinv_backward_issue(c, p.J, finish_tc, head);
  }
  ctx_close(c, kBwdTmemCols);
  NS_TRACE();
#ifdef FNB_NS_TRACE
  if (threadIdx.x == 0 && blockIdx.x < 64) g_ns_span[2 * blockIdx.x + 1] = global_ns();
#endif
}

}  // namespace nstc
}  // namespace fnb
