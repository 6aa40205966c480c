// Host side of the tensor-core path: TMA tensor maps, tile schedule, launches.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <mutex>
#include "tc_stream.cuh"

namespace fnb {
namespace tc {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

// The driver entry point is resolved through the runtime, so the library does not link libcuda.
inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

inline CUtensorMapDataType map_dtype(int dtype) {
  return dtype == FNB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}

// Where slice (b, h) of a (B, H, N, D) tensor lives.  FNB_LAYOUT_BHND: contiguous (B, H, N, D).
// FNB_LAYOUT_BNHD: the head-split view of a contiguous (B, N, H * D) tensor, i.e. rows of one slice
// are H * D elements apart.  The kernels always see a 4-D map (D, N, H', B') and address slice bh as
// (bh % H', bh / H'); for the contiguous layout H' = B * H and B' = 1.
struct BigLayout {
  int64_t B, H, N;
  int D, layout;
  int map_h() const { return layout == FNB_LAYOUT_BNHD ? (int)H : (int)(B * H); }
  int64_t row_stride() const { return layout == FNB_LAYOUT_BNHD ? H * D : D; }                 // elements
  int64_t head_stride() const { return layout == FNB_LAYOUT_BNHD ? D : N * D; }
  int64_t batch_stride() const { return layout == FNB_LAYOUT_BNHD ? N * H * D : H * N * D; }
};

// 16-bit (B, H, N, D) tensor in either layout, box = 64 columns x box_rows rows of one slice,
// 128-byte swizzle.  Rows past N read as zero and are clipped on store.
inline bool make_map_big(CUtensorMap* map, const void* ptr, int dtype, const BigLayout& g, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const bool split = g.layout == FNB_LAYOUT_BNHD;
  cuuint64_t dims[4] = {(cuuint64_t)g.D, (cuuint64_t)g.N, (cuuint64_t)(split ? g.H : g.B * g.H), (cuuint64_t)(split ? g.B : 1)};
  cuuint64_t strides[3] = {(cuuint64_t)g.row_stride() * 2, (cuuint64_t)g.head_stride() * 2,
                           (cuuint64_t)(split ? g.batch_stride() : g.B * g.H * g.N * g.D) * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return fn(map, map_dtype(dtype), 4, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// (rows, cols) 16-bit matrix, box = 64 columns x box_rows rows, 128-byte swizzle.
inline bool make_map_2d(CUtensorMap* map, const void* ptr, int dtype, int64_t rows, int cols, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, map_dtype(dtype), 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// One wave: at most `slots` CTAs (co-resident CTAs per SM x SM count) in total, so that no CTA
// waits for a slot while the others are already done.  Slices are cut into equal runs of tiles.
inline TcSched make_sched(int64_t BH, int64_t N, int slots) {
  TcSched s;
  s.N = N;
  s.seg_N = N;
  s.row_offset = 0;
  s.order = 0;
  s.hint = 0;
  s.test_drop = 0;
  s.H = (int)BH;
  int64_t tiles = (N + kTile - 1) / kTile;
  int64_t want = slots / BH;            // floor: BH * want <= slots
  if (want > tiles) want = tiles;
  if (want < 1) want = 1;
  int64_t tpc = (tiles + want - 1) / want;
  s.tiles_per_chunk = (int)tpc;
  s.nchunk = (int)((tiles + tpc - 1) / tpc);
  return s;
}

inline bool tc_supported(int dtype, int D, int m, uint32_t flags) {
  if (flags & FNB_FLAG_FORCE_GENERIC) return false;
  if (dtype != FNB_F16 && dtype != FNB_BF16) return false;
  return (D == 64 && m <= 64) || (D == 128 && m <= 128);
}

}  // namespace tc
}  // namespace fnb
