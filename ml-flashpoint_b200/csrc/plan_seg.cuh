// Segment table entry of a copy plan and the tile constants shared by the planner and the kernels.
#ifndef MLF_PLAN_SEG_CUH_
#define MLF_PLAN_SEG_CUH_

#include <stdint.h>

#include "mlf_b200.h"

namespace mlf {
namespace plan {

constexpr uint32_t kThreads = 256;
constexpr uint64_t kTileBytes = 64 * 1024;    // FLAT tile and ROWS chunk
#ifndef MLF_ROW_SPLIT_KIB
#define MLF_ROW_SPLIT_KIB 8
#endif
constexpr uint64_t kRowSplitBytes = MLF_ROW_SPLIT_KIB * 1024;  // rows at least this long are linear tiles (cut into 64 KiB chunks)
constexpr int kTransCols = 32;                // TRANSPOSE tile: elements along the tensor-contiguous dim
constexpr int kTransSmemBytes = 32 * 264 + 16;  // 32 rows at the widest pitch + slack for vector reads
constexpr uint64_t kGenericTile = 4096;       // GENERIC elements per tile
constexpr uint64_t kRowsPerTileMax = 64;      // short ROWS: at most this many rows per tile (8 per warp)

enum SegKind : uint32_t { kFlat = 0, kRows = 1, kTranspose = 2, kGeneric = 3 };

struct Seg {
  uint64_t tensor;     // byte address of element 0
  uint64_t image_off;  // byte offset of element 0 in the image
  uint64_t a;          // FLAT: bytes | ROWS: row bytes | TRANSPOSE: tiles per batch | GENERIC: elements
  uint32_t kind;
  uint32_t esize;
  uint32_t ndim;
  uint32_t b;  // FLAT: destination address mod 128 | ROWS: rows per tile (0 = chunked rows) | TRANSPOSE: tiles along L
  uint32_t c;  // ROWS: chunks per row                   | TRANSPOSE: index of dimension C
  uint32_t image_aligned;  // 1 if every image element address is a multiple of esize
  uint32_t d;  // TRANSPOSE: image rows per sub-tile when sub-tiles span whole image rows (0 = wide rows)
  // TRANSPOSE, form of the tile. Narrow rows (d != 0): 0 element-wise walk, 1 the rows are contiguous in the
  // tensor too (no transposition), 7 granules through the cp.async pipeline. Wide rows (d == 0): 0 element-wise,
  // 2 vector form, 4 / 6 matrix form fed by 16-byte / 4-byte cp.async, 5 matrix form behind a register shift.
  uint32_t reserved;
  int64_t shape[MLF_MAX_DIMS];
  int64_t tstride[MLF_MAX_DIMS];  // bytes
  int64_t istride[MLF_MAX_DIMS];  // bytes
};


template <typename T>
__device__ __forceinline__ T load_elem(const uint8_t* p, bool aligned) {
  if (aligned) return *reinterpret_cast<const T*>(p);
  T v;
  uint8_t* b = reinterpret_cast<uint8_t*>(&v);
#pragma unroll
  for (int k = 0; k < (int)sizeof(T); ++k) b[k] = p[k];
  return v;
}
template <typename T>
__device__ __forceinline__ void store_elem(uint8_t* p, T v, bool aligned) {
  if (aligned) {
    *reinterpret_cast<T*>(p) = v;
    return;
  }
  const uint8_t* b = reinterpret_cast<const uint8_t*>(&v);
#pragma unroll
  for (int k = 0; k < (int)sizeof(T); ++k) p[k] = b[k];
}

}  // namespace plan
}  // namespace mlf
#endif  // MLF_PLAN_SEG_CUH_
