// Copy plans: the gather-pack (save) and scatter-unpack (restore) kernel and its host planner.
//
// A plan turns a list of N-d box copies between tensors and one checkpoint-object image into a
// table of segments plus a tile index, uploads both once, and then runs as a single persistent
// kernel per object: CTAs stride over the tiles, find the owning segment with a binary search
// over the tile prefix, and move that tile. Four segment kinds exist:
//   FLAT       both sides contiguous: 64 KiB byte runs, destination-aligned 16-byte vectors
//   ROWS       innermost dimension contiguous on both sides: runs per row (or per row chunk); short
//              rows share a ring slot, one bulk load each
//   TRANSPOSE  the tensor's unit-stride dimension is not the image's: sub-tiles of 32 elements by 256
//              bytes through shared memory so both sides are touched along their contiguous direction,
//              the loads of one sub-tile in flight while the previous one is written out
//   GENERIC    anything else (stepped slices, expands): one element per thread
// FLAT and ROWS tiles stream through a shared-memory ring fed by bulk copies (the streaming phase);
// the table lists their segments first. The image side has byte alignment only, because the object
// format is unpadded.
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <mutex>
#include <string>
#include <vector>

#include "bulk_pipeline.cuh"
#include "common.h"
#include "copy_device.cuh"

namespace {

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
  uint32_t d;  // TRANSPOSE: image rows per sub-tile when sub-tiles span whole image rows (0 = 32-row sub-tiles)
  uint32_t reserved;  // TRANSPOSE with d != 0: 1 = the rows are contiguous in the tensor too (no transposition)
  int64_t shape[MLF_MAX_DIMS];
  int64_t tstride[MLF_MAX_DIMS];  // bytes
  int64_t istride[MLF_MAX_DIMS];  // bytes
};

// ------------------------------------------------------------------------------------ device

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

// Geometry of a TRANSPOSE tile for elements of E bytes (shared by the planner and the kernel).
// A tile is kTransSub sub-tiles that a CTA of kThreads threads moves one after the other through
// one shared-memory staging area, software-pipelined: the global loads of sub-tile j+1 are in
// flight while sub-tile j is written out.
//   wide rows   : a sub-tile is 32 elements along C (contiguous in the tensor) by kRowBytes along L
//                 (contiguous in the image); the sub-tiles of a tile follow one another along L
//   narrow rows : image rows shorter than kRowBytes lying back to back; a sub-tile is as many whole
//                 rows as fit kNarrowBytes, i.e. ONE contiguous run of the image
#ifndef MLF_TRANSPOSE_ATTR
#define MLF_TRANSPOSE_ATTR __noinline__
#endif
constexpr int kTransSub = 4;
template <int E>
struct TransGeom {
  static constexpr int kRowBytes = E == 1 ? 128 : 256;
  static constexpr int kRowElems = kRowBytes / E;
  static constexpr int kPitch = E == 8 ? kRowBytes + 8 : kRowBytes + 4;  // odd word count: columns spread over banks
  static constexpr int kPerThread = kRowElems * kTransCols / (int)kThreads;  // 16, 16, 8, 4
  static constexpr int kNarrowBytes = E == 1 ? 4096 : 8192;
  static constexpr int kNarrowPerThread = kNarrowBytes / E / (int)kThreads;  // 16, 16, 8, 4
  static constexpr int kWordsPerRow = kRowBytes / 4;
  static constexpr int kRowsPerPass = (int)kThreads / kWordsPerRow;
  static constexpr int kPasses = kTransCols / kRowsPerPass;  // 4 or 8
  static constexpr int kNarrowWordsPerThread = kNarrowBytes / 4 / (int)kThreads;  // 4 or 8
};
inline uint32_t trans_row_bytes(uint32_t esize) { return esize == 1 ? 128u : 256u; }
inline uint32_t trans_narrow_bytes(uint32_t esize) { return esize == 1 ? 4096u : 8192u; }

// Misaligned global words -> aligned shared-memory words: word i of the run that starts at
// `gsrc` (any alignment). Callers load lo/hi for a batch of words first and combine afterwards.
__device__ __forceinline__ void ld_word_pair(const uint8_t* gsrc, uint32_t i, bool ok, uint32_t* lo, uint32_t* hi) {
  const uint32_t m = (uint32_t)((uintptr_t)gsrc & 3u);
  const uint32_t* a = reinterpret_cast<const uint32_t*>(gsrc - m);
  *lo = ok ? __ldg(a + i) : 0u;
  *hi = (ok && m) ? __ldg(a + i + 1) : 0u;
}
__device__ __forceinline__ uint32_t join_word_pair(const uint8_t* gsrc, uint32_t lo, uint32_t hi) {
  return __funnelshift_r(lo, hi, 8u * (uint32_t)((uintptr_t)gsrc & 3u));
}

// Shared-memory swizzle of the narrow-row staging area: byte offset -> byte offset with the
// 16-byte granule index inside each 128-byte line XORed with the line number. Image rows of 64 or
// 128 bytes would otherwise put a whole warp's column accesses on one bank.
__device__ __forceinline__ uint32_t swz(uint32_t off) { return off ^ ((off >> 3) & 0x70u); }

// drain_slot for a swizzled staging area: staged byte k (logical offset) goes to dst[k].
__device__ __forceinline__ void drain_swizzled(uint8_t* __restrict__ dst, const uint8_t* __restrict__ staged, uint32_t len,
                                               unsigned tid, unsigned nthr) {
  const uint32_t head = min((16u - (uint32_t)((uintptr_t)dst & 15u)) & 15u, len);
  if (tid < head) dst[tid] = staged[swz(tid)];
  const uint32_t nvec = (len - head) >> 4;
  uint4* __restrict__ d4 = reinterpret_cast<uint4*>(dst + head);
  auto granule = [&](uint32_t v) { return *reinterpret_cast<const uint4*>(staged + swz(v << 4)); };
  if (head == 0) {
#pragma unroll 4
    for (uint32_t i = tid; i < nvec; i += nthr) mlf::st_vec(d4 + i, granule(i));
  } else {
#pragma unroll 4
    for (uint32_t i = tid; i < nvec; i += nthr) mlf::st_vec(d4 + i, mlf::realign(granule(i), granule(i + 1), head));
  }
  const uint32_t tail = (len - head) & 15u;
  if (tid < tail) {
    const uint32_t o = head + (nvec << 4) + tid;
    dst[o] = staged[swz(o)];
  }
}

// Vector form of the wide TRANSPOSE tile (pack direction; segments planned with g.reserved == 2,
// bulk kernels only). The tensor side is read as aligned 16-byte granules instead of single elements:
// per tensor row (fixed l) a tile takes 8 granules = 128 bytes along C and delivers the 112 bytes
// that are complete behind any misalignment of the row start (7 granules after the shift), so a
// warp-wide access covers four rows of 128 contiguous bytes whatever the element size. A sub-tile is
// 128 elements along L: image row segments of 128 * E bytes. Staging is in image order, one row
// per C index, pitch 128 * E + 4.
template <int E>
struct TransV {
  static constexpr int kOutBytes = 112;
  static constexpr int kC = kOutBytes / E;       // image rows per tile: 112, 56, 28, 14
  static constexpr int kL = 128;                 // elements along L per sub-tile
  static constexpr int kRowBytes = kL * E;       // one image row segment
  static constexpr int kPitch = E == 8 ? kRowBytes + 8 : kRowBytes + 4;  // keeps elements aligned, spreads rows over banks
  static constexpr int kPer = 16 / E;            // elements per granule
  static constexpr int kDrainLanes = kRowBytes / 16 >= 32 ? 32 : 16;  // lanes that share one image row in the drain
};
constexpr int kTransVSmemBytes = 112 * (128 + 4) + 32;  // widest case (E = 1); fits one ring slot
inline uint32_t trans_v_cols(uint32_t esize) { return 112u / esize; }
constexpr int kTransVL = 128;

template <typename T>
__device__ __forceinline__ T granule_elem(const uint4& v, int e) {
  constexpr int E = (int)sizeof(T);
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  if (E == 8) return (T)(((uint64_t)w[2 * e + 1] << 32) | w[2 * e]);
  if (E == 4) return (T)w[e];
  if (E == 2) return (T)((w[e >> 1] >> ((e & 1) * 16)) & 0xffffu);
  return (T)((w[e >> 2] >> ((e & 3) * 8)) & 0xffu);
}

// Wide TRANSPOSE tile, vector form. `smem` must hold kTransVSmemBytes. Must run with kThreads threads.
template <typename T, int DIR>
__device__ __noinline__ void transpose_tile_v(const Seg& g, uint32_t local, uint8_t* image, uint8_t* smem) {
  constexpr int E = (int)sizeof(T);
  using V = TransV<E>;
  const int L = (int)g.ndim - 1;
  const int C = (int)g.c;
  const uint32_t tiles_per_batch = (uint32_t)g.a;
  uint64_t batch = local / tiles_per_batch;
  const uint32_t in_batch = local % tiles_per_batch;
  int64_t toff = 0, ioff = 0;
  for (int d = L - 1; d >= 0; --d) {
    if (d == C) continue;
    const int64_t idx = (int64_t)(batch % (uint64_t)g.shape[d]);
    batch /= (uint64_t)g.shape[d];
    toff += idx * g.tstride[d];
    ioff += idx * g.istride[d];
  }
  const int64_t nC = g.shape[C], nL = g.shape[L];
  const int64_t tsL = g.tstride[L], isC = g.istride[C];
  const int64_t c0 = (int64_t)(in_batch / g.b) * V::kC;
  const int64_t lfirst = (int64_t)(in_batch % g.b) * (V::kL * kTransSub);
  const int nsub = (int)min((int64_t)kTransSub, (nL - lfirst + V::kL - 1) / V::kL);
  const int nc = (int)min((int64_t)V::kC, nC - c0);  // image rows of this tile
  const uint32_t row_bytes = (uint32_t)nc * E;       // bytes of each tensor row that belong to the tile
  uint8_t* trow0 = reinterpret_cast<uint8_t*>(g.tensor) + toff + c0 * (int64_t)E + lfirst * tsL;  // tensor row lfirst
  uint8_t* ibase = image + g.image_off + ioff + c0 * isC + lfirst * (int64_t)E;                    // image row c0 at lfirst
  const unsigned tid = threadIdx.x;
  const unsigned j = tid & 7u, lr = tid >> 3;  // granule within the row; row within a pass of 32 rows
  auto elems_of = [&](int s) { return (int)min((int64_t)V::kL, nL - (lfirst + (int64_t)s * V::kL)); };

  static_assert(DIR == MLF_PACK, "the vector form exists for the pack direction only");
  {
    uint4 v[4];
    auto load = [&](int s) {
      const int nl = elems_of(s);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int l = (int)lr + 32 * k;
        const uint8_t* row = trow0 + ((int64_t)s * V::kL + l) * tsL;
        const uint32_t m = (uint32_t)((uintptr_t)row & 15u);
        // only granules that hold at least one byte of the row are touched
        const bool need = l < nl && 16u * j < m + row_bytes;
        v[k] = need ? mlf::ld_vec(reinterpret_cast<const uint4*>(row - m) + j) : make_uint4(0u, 0u, 0u, 0u);
      }
    };
    load(0);
    for (int s = 0; s < nsub; ++s) {
      const int nl = elems_of(s);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int l = (int)lr + 32 * k;
        const uint8_t* row = trow0 + ((int64_t)s * V::kL + l) * tsL;
        const uint32_t m = (uint32_t)((uintptr_t)row & 15u);
        const uint4 next = mlf::shfl_down1(v[k]);  // granule j + 1 of the same row (lanes 8r .. 8r + 7 share a row)
        const uint4 out = m ? mlf::realign(v[k], next, m) : v[k];  // row bytes [16 j, 16 j + 16)
        if (j < 7u && l < nl) {
#pragma unroll
          for (int e = 0; e < V::kPer; ++e) {
            const int c = (int)j * V::kPer + e;
            if (c < nc) *reinterpret_cast<T*>(smem + c * V::kPitch + l * E) = granule_elem<T>(out, e);
          }
        }
      }
      __syncthreads();
      if (s + 1 < nsub) load(s + 1);
      uint8_t* irow = ibase + (int64_t)s * V::kL * E;
      constexpr unsigned DL = (unsigned)V::kDrainLanes;
      for (unsigned r = tid / DL; r < (unsigned)nc; r += kThreads / DL) {
        const uint32_t at = r * (uint32_t)V::kPitch;
        mlf::drain_slot(irow + (int64_t)r * isC, smem + (at & ~15u), at & 15u, (uint32_t)nl * E, tid % DL, DL);
      }
      __syncthreads();
    }
  }
}

// cp.async and shared-memory helpers of the staged transposes.
// Shared-memory accesses by 32-bit shared-window address (mlf::smem_addr): the staged transposes
// compute many addresses per byte moved, and these keep that arithmetic in 32 bits.
__device__ __forceinline__ void sts_b8(uint32_t a, uint32_t v) { asm volatile("st.shared.b8 [%0], %1;" ::"r"(a), "h"((uint16_t)v) : "memory"); }
__device__ __forceinline__ void sts_b16(uint32_t a, uint32_t v) { asm volatile("st.shared.b16 [%0], %1;" ::"r"(a), "h"((uint16_t)v) : "memory"); }
__device__ __forceinline__ void sts_b32(uint32_t a, uint32_t v) { asm volatile("st.shared.b32 [%0], %1;" ::"r"(a), "r"(v) : "memory"); }
__device__ __forceinline__ void sts_b64(uint32_t a, uint32_t lo, uint32_t hi) {
  asm volatile("st.shared.v2.b32 [%0], {%1,%2};" ::"r"(a), "r"(lo), "r"(hi) : "memory");
}
__device__ __forceinline__ void sts_b128(uint32_t a, const uint4& v) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 lds_b128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ uint8_t lds_b8(uint32_t a) {
  uint16_t v;
  asm volatile("ld.shared.u8 %0, [%1];" : "=h"(v) : "r"(a) : "memory");
  return (uint8_t)v;
}
__device__ __forceinline__ void cp_async16_at(uint32_t smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async4_at(uint32_t smem_dst, const void* gmem_src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Matrix form of the wide TRANSPOSE tile: 16- and 32-bit elements, pack direction, tensor rows that
// all start on 16-byte boundaries (segments planned with g.reserved == 4, bulk kernels only). Stages
// of 128 tensor rows by 128 bytes arrive by cp.async, two deep, granules XOR-swizzled so that the
// warp-level matrix loads below are conflict-free. One ldmatrix.x4.trans per warp turns a block of
// 32 rows by one granule into registers that hold, per thread, CONSECUTIVE elements of one image
// row: the four 8x8 matrices of 16-bit values are given interleaved row lists for exactly that
// (32-bit elements arrive as their two halves in neighbouring threads and are put together with one
// shuffle and one byte permute per register). Each thread then owns one aligned 16-byte piece of an
// image row, which goes to an image-order staging area with a single conflict-free 16-byte
// shared-memory store. The staging rows are written out as aligned 16-byte image vectors, shifted by
// the image's byte misalignment; vectors that straddle two stages take their leading bytes from a
// per-row carry, so only the two ends of a tile's image rows are written bytewise.
template <int E>
struct TransM {
  static constexpr int kCols = 128 / E;            // elements along C per tile: 64 or 32 (128 bytes of each tensor row)
  static constexpr int kSegBytes = 128 * E;        // bytes of one image row per full stage: 256 or 512
  static constexpr int kPitch = kSegBytes + 64;    // image-order staging row; pitch = 4 mod 8 granules
  static constexpr int kPositions = kSegBytes / 16;  // aligned image vectors per row and stage
  static constexpr int kCarryBytes = kCols * 16;   // per parity
};
constexpr int kTransML = 128;       // tensor rows per stage
#ifndef MLF_TRANSM_SUB
#define MLF_TRANSM_SUB 8
#endif
constexpr int kTransMSub = MLF_TRANSM_SUB;  // stages per tile
constexpr int kTransMStageBytes = kTransML * 128;      // 16 KiB, tensor order
constexpr int kTransMStagingOff = 2 * kTransMStageBytes;
inline uint32_t trans_m_cols(uint32_t esize) { return 128u / esize; }

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_row));
}
// Position of granule g of tensor row l inside its 128-byte stage row. The key takes the bits of l
// in which the eight rows of one 8x8 matrix differ (see the row lists in transpose_tile_m).
template <int E>
__device__ __forceinline__ uint32_t matrix_swizzle(uint32_t l, uint32_t g) {
  const uint32_t key = (((l >> 3) & 3u) << 1) | (E == 2 ? (l & 1u) : ((l >> 2) & 1u));
  return (g ^ key) << 4;
}

// `ring`: two tensor-order stages, then the image-order staging area; `aux`: two parities of carries.
// WORDS: the tensor rows start on 4-byte instead of 16-byte boundaries; the stages are then fed by
// 4-byte cp.async copies (a warp covers one row's 128 bytes per instruction), which land every row
// at the start of its stage row whatever its alignment in global memory.
template <int E, bool WORDS>
__device__ __noinline__ void transpose_tile_m(const Seg& g, uint32_t local, uint8_t* image, uint8_t* ring, uint8_t* aux) {
  using M = TransM<E>;
  const int L = (int)g.ndim - 1;
  const int C = (int)g.c;
  const uint32_t tiles_per_batch = (uint32_t)g.a;
  uint64_t batch = local / tiles_per_batch;
  const uint32_t in_batch = local % tiles_per_batch;
  int64_t toff = 0, ioff = 0;
  for (int d = L - 1; d >= 0; --d) {
    if (d == C) continue;
    const int64_t idx = (int64_t)(batch % (uint64_t)g.shape[d]);
    batch /= (uint64_t)g.shape[d];
    toff += idx * g.tstride[d];
    ioff += idx * g.istride[d];
  }
  const int64_t nC = g.shape[C], nL = g.shape[L];
  const int64_t tsL = g.tstride[L], isC = g.istride[C];
  const int64_t c0 = (int64_t)(in_batch / g.b) * M::kCols;
  const int64_t lfirst = (int64_t)(in_batch % g.b) * (kTransML * kTransMSub);
  const int nsub = (int)min((int64_t)kTransMSub, (nL - lfirst + kTransML - 1) / kTransML);
  const int nc = (int)min((int64_t)M::kCols, nC - c0);
  const uint32_t row_bytes = (uint32_t)nc * E;
  const uint8_t* trow0 = reinterpret_cast<const uint8_t*>(g.tensor) + toff + c0 * (int64_t)E + lfirst * tsL;  // 16-byte aligned
  uint8_t* ibase = image + g.image_off + ioff + c0 * isC + lfirst * (int64_t)E;
  const unsigned tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
  const uint32_t ring_at = mlf::smem_addr(ring), aux_at = mlf::smem_addr(aux);
  const uint32_t staging = ring_at + kTransMStagingOff;  // shared-window addresses from here on
  auto elems_of = [&](int s) { return (int)min((int64_t)kTransML, nL - (lfirst + (int64_t)s * kTransML)); };

  auto issue = [&](int s) {
    const int nl = elems_of(s);
    const uint32_t stage = ring_at + (uint32_t)(s & 1) * kTransMStageBytes;
    if (WORDS) {
      const unsigned w = tid & 31u, lr = tid >> 5;  // word within the row; row within a pass of 8 rows
#pragma unroll 4
      for (int k = 0; k < 16; ++k) {
        const unsigned l = lr + 8u * k;
        if ((int)l < nl && 4u * w < row_bytes)
          cp_async4_at(stage + l * 128u + matrix_swizzle<E>(l, w >> 2) + 4u * (w & 3u), trow0 + ((int64_t)s * kTransML + l) * tsL + 4u * w);
      }
    } else {
      const unsigned gq = tid & 7u, lr = tid >> 3;  // granule within the row; row within a pass of 32 rows
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const unsigned l = lr + 32u * k;
        if ((int)l < nl && 16u * gq < row_bytes)
          cp_async16_at(stage + l * 128u + matrix_swizzle<E>(l, gq), trow0 + ((int64_t)s * kTransML + l) * tsL + 16u * gq);
      }
    }
    cp_async_commit();
  };

  issue(0);
  if (nsub > 1) issue(1); else cp_async_commit();
  for (int s = 0; s < nsub; ++s) {
    if (s + 1 < nsub) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();  // stage s has landed; every thread is done draining the staging area of stage s - 1
    const int nl = elems_of(s);
    const int seg_len = nl * E;
    const bool first = s == 0, last = s == nsub - 1;
    const uint32_t stage = ring_at + (uint32_t)(s & 1) * kTransMStageBytes;
    // ---- transpose: blocks of 32 tensor rows by one granule, four per warp
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const unsigned blk = warp + 8u * b, lb = blk >> 3, cb = blk & 7u;
      // lane = 8 i + k supplies row k of matrix i. A thread receives rows 2 t and 2 t + 1 (t = lane % 4)
      // of every matrix, so the row lists are laid out for its four registers to be consecutive
      // elements of one image row:
      //   16-bit: row(i, k) = 32 lb + 8 (k / 2) + 2 i + k % 2        -> registers hold l = 8 t + 0 .. 7
      //   32-bit: row(i, k) = 32 lb + 8 (k / 2) + i + 4 (k % 2)      -> after the exchange: l = 8 t + 4 p + 0 .. 3
      const unsigned i = lane >> 3, k = lane & 7u;
      const unsigned l = 32u * lb + 8u * (k >> 1) + (E == 2 ? 2u * i + (k & 1u) : i + 4u * (k & 1u));
      uint32_t r[4];
      ldmatrix_x4_trans(r, stage + l * 128u + matrix_swizzle<E>(l, cb));
      const unsigned t = lane & 3u;
      if (E == 2) {
        // image row 8 cb + lane / 4, elements 32 lb + 8 t .. + 7
        const unsigned c = 8u * cb + (lane >> 2), l0 = 32u * lb + 8u * t;
        sts_b128(staging + c * M::kPitch + l0 * E, make_uint4(r[0], r[1], r[2], r[3]));
      } else {
        // the two halves of a 32-bit element sit in this thread and in lane ^ 4: the thread with the
        // low halves (p = 0) assembles the element of row 2 t, its neighbour that of row 2 t + 1
        const unsigned p = (lane >> 2) & 1u;
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t other = __shfl_xor_sync(0xffffffffu, r[q], 4);
          o[q] = p ? __byte_perm(other, r[q], 0x7632) : __byte_perm(r[q], other, 0x5410);
        }
        const unsigned c = 4u * cb + (lane >> 3), l0 = 32u * lb + 8u * t + 4u * p;
        sts_b128(staging + c * M::kPitch + l0 * E, make_uint4(o[0], o[1], o[2], o[3]));
      }
    }
    __syncthreads();  // staging holds the stage in image order; the tensor-order buffer is free again
    if (s + 2 < nsub) issue(s + 2); else cp_async_commit();
    // ---- write out: aligned 16-byte image vectors, kPositions per image row. With a misaligned row
    // (h != 0) the first position straddles in from the previous stage and the row's last 16 - h
    // bytes wait in the carry, so the count is the same.
    const uint32_t carry_in = aux_at + (uint32_t)((s + 1) & 1) * M::kCarryBytes;  // last 16 bytes of stage s - 1 per image row
    const uint32_t carry_out = aux_at + (uint32_t)(s & 1) * M::kCarryBytes;
    uint8_t* iseg = ibase + (int64_t)s * M::kSegBytes;
    // 16 lanes per image row (a warp-wide store covers two rows of 256 contiguous bytes)
    for (int c = (int)(tid >> 4); c < nc; c += (int)(kThreads >> 4)) {
      uint8_t* row = iseg + (int64_t)c * isC;
      const uint32_t data = staging + (uint32_t)c * M::kPitch;
      const int h = (int)((16u - (uint32_t)((uintptr_t)row & 15u)) & 15u);  // the same in every stage
#pragma unroll
      for (int j = 0; j < M::kPositions / 16; ++j) {
        const int vq = (int)(tid & 15u) + 16 * j;
        if (h == 0) {
          if (16 * (vq + 1) <= seg_len) mlf::st_vec(reinterpret_cast<uint4*>(row + 16 * vq), lds_b128(data + 16u * vq));
        } else {
          const int q = h - 16 + 16 * vq;  // stage-relative first byte of the vector
          if (q + 16 <= seg_len && !(first && vq == 0)) {
            const uint4 lo = lds_b128(vq == 0 ? carry_in + (uint32_t)c * 16u : data + 16u * (vq - 1));
            const uint4 hi = lds_b128(data + 16u * vq);
            mlf::st_vec(reinterpret_cast<uint4*>(row + q), mlf::realign(lo, hi, (unsigned)h));
          }
        }
      }
    }
    if (!last && (int)tid < nc)
      sts_b128(carry_out + tid * 16u, lds_b128(staging + tid * M::kPitch + M::kSegBytes - 16));
    if (first) {
      for (int idx = (int)tid; idx < nc * 15; idx += (int)kThreads) {
        const int c = idx / 15, kb = idx % 15;
        uint8_t* row = iseg + (int64_t)c * isC;
        const int h = (int)((16u - (uint32_t)((uintptr_t)row & 15u)) & 15u);
        if (kb < h && kb < seg_len) row[kb] = lds_b8(staging + (uint32_t)(c * M::kPitch + kb));
      }
    }
    if (last) {
      for (int idx = (int)tid; idx < nc * 15; idx += (int)kThreads) {
        const int c = idx / 15, kb = idx % 15;
        uint8_t* row = iseg + (int64_t)c * isC;
        const int h = (int)((16u - (uint32_t)((uintptr_t)row & 15u)) & 15u);
        int done = seg_len - (int)(((uintptr_t)row + (uint32_t)seg_len) & 15u);  // last 16-byte boundary of the image inside the segment
        if (first && done < h) done = min(h, seg_len);
        const int b = done + kb;
        if (b >= seg_len || (first && b < h)) continue;
        if (b >= 0)
          row[b] = lds_b8(staging + (uint32_t)(c * M::kPitch + b));
        else if (!first)
          row[b] = lds_b8(carry_in + (uint32_t)(c * 16 + 16 + b));
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();  // the staging area and the carries are free for the next tile
}

// Matrix form for tensor rows that start anywhere (segments planned with g.reserved == 5): the same
// transposition and write-out as transpose_tile_m, but the tensor rows are read the way the vector
// form reads them, as aligned granules through registers (one stage ahead), shifted into place with
// shf.r and then stored, 16 bytes at a time, into the swizzled tensor-order stage. A tile row
// delivers the 112 bytes (7 granules) that are complete behind any shift.
template <int E>
struct TransMS {
  static constexpr int kCols = 112 / E;            // 56 or 28 image rows per tile
  static constexpr int kGranules = 7;
  static constexpr int kSegBytes = 128 * E;
  static constexpr int kPitch = kSegBytes + 64;
  static constexpr int kPositions = kSegBytes / 16;
  static constexpr int kCarryBytes = kCols * 16;
};
inline uint32_t trans_ms_cols(uint32_t esize) { return 112u / esize; }

// `ring`: one tensor-order stage (16 KiB), then (at kTransMStagingOff) the image-order staging area.
template <int E>
__device__ __noinline__ void transpose_tile_ms(const Seg& g, uint32_t local, uint8_t* image, uint8_t* ring, uint8_t* aux) {
  using M = TransMS<E>;
  const int L = (int)g.ndim - 1;
  const int C = (int)g.c;
  const uint32_t tiles_per_batch = (uint32_t)g.a;
  uint64_t batch = local / tiles_per_batch;
  const uint32_t in_batch = local % tiles_per_batch;
  int64_t toff = 0, ioff = 0;
  for (int d = L - 1; d >= 0; --d) {
    if (d == C) continue;
    const int64_t idx = (int64_t)(batch % (uint64_t)g.shape[d]);
    batch /= (uint64_t)g.shape[d];
    toff += idx * g.tstride[d];
    ioff += idx * g.istride[d];
  }
  const int64_t nC = g.shape[C], nL = g.shape[L];
  const int64_t tsL = g.tstride[L], isC = g.istride[C];
  const int64_t c0 = (int64_t)(in_batch / g.b) * M::kCols;
  const int64_t lfirst = (int64_t)(in_batch % g.b) * (kTransML * kTransMSub);
  const int nsub = (int)min((int64_t)kTransMSub, (nL - lfirst + kTransML - 1) / kTransML);
  const int nc = (int)min((int64_t)M::kCols, nC - c0);
  const uint32_t row_bytes = (uint32_t)nc * E;
  const uint8_t* trow0 = reinterpret_cast<const uint8_t*>(g.tensor) + toff + c0 * (int64_t)E + lfirst * tsL;
  uint8_t* ibase = image + g.image_off + ioff + c0 * isC + lfirst * (int64_t)E;
  const unsigned tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
  const uint32_t stage = mlf::smem_addr(ring), aux_at = mlf::smem_addr(aux);  // shared-window addresses from here on
  const uint32_t staging = stage + kTransMStagingOff;
  auto elems_of = [&](int s) { return (int)min((int64_t)kTransML, nL - (lfirst + (int64_t)s * kTransML)); };
  const unsigned gq = tid & 7u, lr = tid >> 3;  // granule within the row; row within a pass of 32 rows

  uint4 v[4];
  auto load = [&](int s) {
    const int nl = elems_of(s);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int l = (int)lr + 32 * k;
      const uint8_t* row = trow0 + ((int64_t)s * kTransML + l) * tsL;
      const uint32_t m = (uint32_t)((uintptr_t)row & 15u);
      const bool need = l < nl && 16u * gq < m + row_bytes;  // only granules that hold at least one byte of the row
      v[k] = need ? mlf::ld_vec(reinterpret_cast<const uint4*>(row - m) + gq) : make_uint4(0u, 0u, 0u, 0u);
    }
  };

  load(0);
  for (int s = 0; s < nsub; ++s) {
    const int nl = elems_of(s);
    const int seg_len = nl * E;
    const bool first = s == 0, last = s == nsub - 1;
    // ---- shift the rows into place and put them into the swizzled stage
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const unsigned l = lr + 32u * k;
      const uint8_t* row = trow0 + ((int64_t)s * kTransML + l) * tsL;
      const uint32_t m = (uint32_t)((uintptr_t)row & 15u);
      const uint4 next = mlf::shfl_down1(v[k]);  // granule gq + 1 of the same row (lanes 8 r .. 8 r + 7 share a row)
      const uint4 out = m ? mlf::realign(v[k], next, m) : v[k];  // row bytes [16 gq, 16 gq + 16)
      if (gq < (unsigned)M::kGranules) sts_b128(stage + l * 128u + matrix_swizzle<E>(l, gq), out);
    }
    __syncthreads();  // the stage is complete; every thread is done draining the staging area of stage s - 1
    if (s + 1 < nsub) load(s + 1);  // in flight while this stage is transposed and written out
    // ---- transpose: blocks of 32 tensor rows by one granule (7 granule columns)
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const unsigned blk = warp + 8u * b;
      if (blk >= 4u * M::kGranules) break;  // warp-uniform
      const unsigned lb = blk / M::kGranules, cb = blk % M::kGranules;
      const unsigned i = lane >> 3, k = lane & 7u;
      const unsigned l = 32u * lb + 8u * (k >> 1) + (E == 2 ? 2u * i + (k & 1u) : i + 4u * (k & 1u));
      uint32_t r[4];
      ldmatrix_x4_trans(r, stage + l * 128u + matrix_swizzle<E>(l, cb));
      const unsigned t = lane & 3u;
      if (E == 2) {
        const unsigned c = 8u * cb + (lane >> 2), l0 = 32u * lb + 8u * t;
        sts_b128(staging + c * M::kPitch + l0 * E, make_uint4(r[0], r[1], r[2], r[3]));
      } else {
        const unsigned p = (lane >> 2) & 1u;
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t other = __shfl_xor_sync(0xffffffffu, r[q], 4);
          o[q] = p ? __byte_perm(other, r[q], 0x7632) : __byte_perm(r[q], other, 0x5410);
        }
        const unsigned c = 4u * cb + (lane >> 3), l0 = 32u * lb + 8u * t + 4u * p;
        sts_b128(staging + c * M::kPitch + l0 * E, make_uint4(o[0], o[1], o[2], o[3]));
      }
    }
    __syncthreads();  // staging holds the stage in image order; the tensor-order stage is free again
    // ---- write out (as in transpose_tile_m)
    const uint32_t carry_in = aux_at + (uint32_t)((s + 1) & 1) * M::kCarryBytes;
    const uint32_t carry_out = aux_at + (uint32_t)(s & 1) * M::kCarryBytes;
    uint8_t* iseg = ibase + (int64_t)s * M::kSegBytes;
    for (int c = (int)(tid >> 4); c < nc; c += (int)(kThreads >> 4)) {
      uint8_t* row = iseg + (int64_t)c * isC;
      const uint32_t data = staging + (uint32_t)c * M::kPitch;
      const int h = (int)((16u - (uint32_t)((uintptr_t)row & 15u)) & 15u);
#pragma unroll
      for (int j = 0; j < M::kPositions / 16; ++j) {
        const int vq = (int)(tid & 15u) + 16 * j;
        if (h == 0) {
          if (16 * (vq + 1) <= seg_len) mlf::st_vec(reinterpret_cast<uint4*>(row + 16 * vq), lds_b128(data + 16u * vq));
        } else {
          const int q = h - 16 + 16 * vq;
          if (q + 16 <= seg_len && !(first && vq == 0)) {
            const uint4 lo = lds_b128(vq == 0 ? carry_in + (uint32_t)c * 16u : data + 16u * (vq - 1));
            const uint4 hi = lds_b128(data + 16u * vq);
            mlf::st_vec(reinterpret_cast<uint4*>(row + q), mlf::realign(lo, hi, (unsigned)h));
          }
        }
      }
    }
    if (!last && (int)tid < nc)
      sts_b128(carry_out + tid * 16u, lds_b128(staging + tid * M::kPitch + M::kSegBytes - 16));
    if (first) {
      for (int idx = (int)tid; idx < nc * 15; idx += (int)kThreads) {
        const int c = idx / 15, kb = idx % 15;
        uint8_t* row = iseg + (int64_t)c * isC;
        const int h = (int)((16u - (uint32_t)((uintptr_t)row & 15u)) & 15u);
        if (kb < h && kb < seg_len) row[kb] = lds_b8(staging + (uint32_t)(c * M::kPitch + kb));
      }
    }
    if (last) {
      for (int idx = (int)tid; idx < nc * 15; idx += (int)kThreads) {
        const int c = idx / 15, kb = idx % 15;
        uint8_t* row = iseg + (int64_t)c * isC;
        const int h = (int)((16u - (uint32_t)((uintptr_t)row & 15u)) & 15u);
        int done = seg_len - (int)(((uintptr_t)row + (uint32_t)seg_len) & 15u);
        if (first && done < h) done = min(h, seg_len);
        const int b = done + kb;
        if (b >= seg_len || (first && b < h)) continue;
        if (b >= 0)
          row[b] = lds_b8(staging + (uint32_t)(c * M::kPitch + b));
        else if (!first)
          row[b] = lds_b8(carry_in + (uint32_t)(c * 16 + 16 + b));
      }
    }
  }
  __syncthreads();  // the staging area and the carries are free for the next tile
}

// drain_swizzled with the staging area given by its shared-window address.
__device__ __forceinline__ void drain_swizzled_at(uint8_t* __restrict__ dst, uint32_t staged, uint32_t len, unsigned tid, unsigned nthr) {
  const uint32_t head = min((16u - (uint32_t)((uintptr_t)dst & 15u)) & 15u, len);
  if (tid < head) dst[tid] = lds_b8(staged + swz(tid));
  const uint32_t nvec = (len - head) >> 4;
  uint4* __restrict__ d4 = reinterpret_cast<uint4*>(dst + head);
  if (head == 0) {
#pragma unroll 4
    for (uint32_t i = tid; i < nvec; i += nthr) mlf::st_vec(d4 + i, lds_b128(staged + swz(i << 4)));
  } else {
#pragma unroll 4
    for (uint32_t i = tid; i < nvec; i += nthr)
      mlf::st_vec(d4 + i, mlf::realign(lds_b128(staged + swz(i << 4)), lds_b128(staged + swz((i + 1) << 4)), head));
  }
  const uint32_t tail = (len - head) & 15u;
  if (tid < tail) {
    const uint32_t o = head + (nvec << 4) + tid;
    dst[o] = lds_b8(staged + swz(o));
  }
}

// Narrow transposed rows, pack direction of the bulk kernels (segments planned with
// g.reserved == 7 and kNarrowASub sub-tiles per tile): sub-tile j holds the image rows
// [cfirst + j d, + d) of nln elements each, one contiguous run of the image, staged in shared memory
// in image order. The tensor side is read in aligned 16-byte granules: granule q of tensor row l
// covers bytes [16 q - m, 16 q - m + 16) of that row's run of d elements, m being the row's
// misalignment. Only granules holding at least one byte of the run are read; elements outside it
// are dropped when the granule is scattered into the staging area. A sub-tile has at most
// narrow_bytes / 16 + 2 nln such granules, which is below 3 kThreads for rows of up to 127 elements.
// The granules arrive by cp.async in stages of their own, kNarrowAStages - 1 sub-tiles ahead; every
// thread reads back exactly the granules it asked for, so a stage needs no barrier. The image-order staging area
// is doubled: while a sub-tile drains, the next one is scattered into the other half, with one
// barrier per sub-tile. `ring`: the stages, then the two staging halves.
constexpr int kNarrowASub = 16;
constexpr int kNarrowAStages = 4;
constexpr int kNarrowAGranules = 3;  // per thread and sub-tile
constexpr int kNarrowAMaxRow = 127;  // elements per image row: 8192 / 16 + 2 * 127 granules at most per sub-tile
constexpr int kNarrowARawBytes = kNarrowAGranules * (int)kThreads * 16;
constexpr int kNarrowAStagingOff = kNarrowAStages * kNarrowARawBytes;
constexpr int kNarrowASmemBytes = kNarrowAStagingOff + 2 * 8192;
template <typename T>
__device__ __noinline__ void transpose_narrow_async(const Seg& g, uint32_t local, uint8_t* image, uint8_t* ring) {
  constexpr int E = (int)sizeof(T);
  constexpr int NG = kNarrowAGranules;
  constexpr int S = kNarrowAStages;
  constexpr int EPG = 16 / E;
  constexpr int LOG_E = E == 1 ? 0 : E == 2 ? 1 : E == 4 ? 2 : 3;
  const int L = (int)g.ndim - 1;
  const int C = (int)g.c;
  const uint32_t tiles_per_batch = (uint32_t)g.a;
  uint64_t batch = local / tiles_per_batch;
  const uint32_t in_batch = local % tiles_per_batch;
  int64_t toff = 0, ioff = 0;
  for (int k = L - 1; k >= 0; --k) {
    if (k == C) continue;
    const int64_t idx = (int64_t)(batch % (uint64_t)g.shape[k]);
    batch /= (uint64_t)g.shape[k];
    toff += idx * g.tstride[k];
    ioff += idx * g.istride[k];
  }
  const uint8_t* tbase = reinterpret_cast<const uint8_t*>(g.tensor) + toff;
  uint8_t* ibase = image + g.image_off + ioff;
  const int64_t nC = g.shape[C], tsL = g.tstride[L], isC = g.istride[C];
  const uint32_t nln = (uint32_t)g.shape[L], d = g.d;
  const int64_t cfirst = (int64_t)in_batch * d * kNarrowASub;
  const int nsub = (int)min((int64_t)kNarrowASub, (nC - cfirst + d - 1) / d);
  const unsigned tid = threadIdx.x;
  const uint32_t step = nln * E;  // staging distance between neighbouring image rows
  auto rows_of = [&](int j) { return (uint32_t)min((int64_t)d, nC - (cfirst + (int64_t)j * d)); };
  // Granule k of this thread is granule gq[k] of tensor row gl[k] in every sub-tile: rows are cut
  // into per_row granules as for a full sub-tile of d image rows; shorter runs leave some unused.
  struct Granule {
    const uint8_t* src;
    int32_t c;  // image row (within the sub-tile) of the first element; may be negative
    bool have;  // the granule holds at least one byte of the run
  };
  const uint32_t per_row = ((d * E + 15u) >> 4) + 1u;
  uint32_t gl[NG], gq[NG];
#pragma unroll
  for (int k = 0; k < NG; ++k) {
    const uint32_t idx = tid + (uint32_t)k * kThreads;
    gl[k] = idx / per_row;
    gq[k] = 16u * (idx - gl[k] * per_row);
  }
  auto granule = [&](int j, int k) {
    const uint32_t run = rows_of(j) * E;
    const uint8_t* row = tbase + (cfirst + (int64_t)j * d) * E + (int64_t)gl[k] * tsL;
    const uint32_t m = (uint32_t)((uintptr_t)row & 15u);
    Granule r;
    r.have = gl[k] < nln && gq[k] < m + run;
    r.src = row - m + gq[k];
    r.c = ((int32_t)gq[k] - (int32_t)m) >> LOG_E;
    return r;
  };
  const uint32_t ring_at = mlf::smem_addr(ring);
  auto issue = [&](int j) {
    const uint32_t raw = ring_at + (uint32_t)(j % S) * kNarrowARawBytes;
#pragma unroll
    for (int k = 0; k < NG; ++k) {
      const Granule r = granule(j, k);
      if (r.have)
        cp_async16_at(raw + (tid + (uint32_t)k * kThreads) * 16u, r.src);
    }
    cp_async_commit();
  };
#pragma unroll
  for (int j = 0; j < S - 1; ++j) {
    if (j < nsub) issue(j); else cp_async_commit();
  }
  for (int j = 0; j < nsub; ++j) {
    if (j + S - 1 < nsub) issue(j + S - 1); else cp_async_commit();
    cp_async_wait<S - 1>();  // this thread's granules of sub-tile j have landed
    const uint32_t raw = ring_at + (uint32_t)(j % S) * kNarrowARawBytes;
    const uint32_t staging = ring_at + kNarrowAStagingOff + (uint32_t)(j & 1) * 8192u;
    const uint32_t ncn = rows_of(j);
    auto put = [&](uint32_t off, const uint32_t (&w)[4], int i) {
      const uint32_t a = staging + swz(off);
      if (E == 8)
        sts_b64(a, w[(2 * i) & 3], w[(2 * i + 1) & 3]);
      else if (E == 4)
        sts_b32(a, w[i & 3]);
      else if (E == 2)
        sts_b16(a, w[(i >> 1) & 3] >> (16 * (i & 1)));
      else
        sts_b8(a, w[(i >> 2) & 3] >> (8 * (i & 3)));
    };
#pragma unroll
    for (int k = 0; k < NG; ++k) {
      const Granule r = granule(j, k);
      if (r.have) {
        const uint4 v = lds_b128(raw + (tid + (uint32_t)k * kThreads) * 16u);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        const uint32_t at = (uint32_t)(r.c * (int32_t)step + (int32_t)(gl[k] * E));
        if (r.c >= 0 && r.c + EPG <= (int32_t)ncn) {  // every element lies in the run
#pragma unroll
          for (int i = 0; i < EPG; ++i) put(at + (uint32_t)i * step, w, i);
        } else {
#pragma unroll
          for (int i = 0; i < EPG; ++i)
            if ((uint32_t)(r.c + i) < ncn) put(at + (uint32_t)i * step, w, i);
        }
      }
    }
    __syncthreads();  // sub-tile j is staged; everyone is done draining sub-tile j - 1
    drain_swizzled_at(ibase + (cfirst + (int64_t)j * d) * isC, staging, ncn * step, tid, kThreads);
  }
  cp_async_wait<0>();
  __syncthreads();  // the stages and the staging halves are free for the next tile
}

// Tile `local` of TRANSPOSE segment g. Must run with kThreads threads.
template <typename T, int DIR>
__device__ MLF_TRANSPOSE_ATTR void transpose_tile(const Seg& g, uint32_t local, uint8_t* image, uint8_t* smem) {
  constexpr int E = (int)sizeof(T);
  using G = TransGeom<E>;
  constexpr int TL = G::kRowElems;
  constexpr int ROW = G::kPitch;
  const int L = (int)g.ndim - 1;
  const int C = (int)g.c;
  const uint32_t tiles_per_batch = (uint32_t)g.a;
  uint64_t batch = local / tiles_per_batch;
  const uint32_t in_batch = local % tiles_per_batch;
  int64_t toff = 0, ioff = 0;
  for (int d = L - 1; d >= 0; --d) {
    if (d == C) continue;
    const int64_t idx = (int64_t)(batch % (uint64_t)g.shape[d]);
    batch /= (uint64_t)g.shape[d];
    toff += idx * g.tstride[d];
    ioff += idx * g.istride[d];
  }
  uint8_t* tbase = reinterpret_cast<uint8_t*>(g.tensor) + toff;
  uint8_t* ibase = image + g.image_off + ioff;
  const int64_t nC = g.shape[C], nL = g.shape[L];
  const int64_t tsL = g.tstride[L], isC = g.istride[C];
  const unsigned tid = threadIdx.x;

  if (g.d != 0) {
    // ---- narrow rows: a sub-tile is g.d whole image rows = one contiguous run of the image,
    // staged in shared memory in image order (16-byte granules swizzled, see swz()). Threads walk
    // the sub-tile's elements along the tensor's unit-stride dimension: element number n is
    // (slow, fast) = (n / nfast, n % nfast), advanced incrementally by kThreads per step.
    //   transposed (g.reserved == 0): fast = image row c, slow = position l in the row
    //   row order  (g.reserved == 1): fast = position in the row, slow = image row
    const bool row_order = g.reserved == 1;
    const uint32_t nln = (uint32_t)nL;
    const int64_t cfirst = (int64_t)in_batch * g.d * kTransSub;
    const int nsub = (int)min((int64_t)kTransSub, (nC - cfirst + g.d - 1) / g.d);
    const int64_t ts_row = g.tstride[C];                 // tensor step between image rows
    const int64_t ts_slow = row_order ? ts_row : tsL;    // tensor step of the walk's slow index
    struct Walk {
      uint32_t slow, fast, dslow, dfast, nfast;
      __device__ __forceinline__ void start(uint32_t n, unsigned t) {
        nfast = n;
        slow = t / n;
        fast = t % n;
        dslow = kThreads / n;
        dfast = kThreads % n;
      }
      __device__ __forceinline__ void next() {
        fast += dfast;
        slow += dslow;
        if (fast >= nfast) {
          fast -= nfast;
          ++slow;
        }
      }
    };
    auto rows_of = [&](int j) { return (uint32_t)min((int64_t)g.d, nC - (cfirst + (int64_t)j * g.d)); };
    auto staged_at = [&](const Walk& w) { return swz((row_order ? w.slow * nln + w.fast : w.fast * nln + w.slow) * E); };
    constexpr int NE = G::kNarrowPerThread;
    if (DIR == MLF_PACK) {
      T v[NE];
      auto load = [&](int j) {
        const uint32_t ncn = rows_of(j), nel = ncn * nln;
        const uint8_t* trun = tbase + (cfirst + (int64_t)j * g.d) * ts_row;
        Walk w;
        w.start(row_order ? nln : ncn, tid);
#pragma unroll
        for (int k = 0; k < NE; ++k) {
          v[k] = (tid + (uint32_t)k * kThreads < nel) ? __ldg(reinterpret_cast<const T*>(trun + (int64_t)w.fast * E + (int64_t)w.slow * ts_slow)) : T(0);
          w.next();
        }
      };
      load(0);
      for (int j = 0; j < nsub; ++j) {
        const uint32_t ncn = rows_of(j), nel = ncn * nln;
        Walk w;
        w.start(row_order ? nln : ncn, tid);
#pragma unroll
        for (int k = 0; k < NE; ++k) {
          if (tid + (uint32_t)k * kThreads < nel) *reinterpret_cast<T*>(smem + staged_at(w)) = v[k];
          w.next();
        }
        __syncthreads();
        if (j + 1 < nsub) load(j + 1);
        drain_swizzled(ibase + (cfirst + (int64_t)j * g.d) * isC, smem, nel * E, tid, kThreads);
        __syncthreads();
      }
    } else {
      constexpr int N = G::kNarrowWordsPerThread;
      uint32_t lo[N], hi[N];
      auto load = [&](int j) {
        const uint8_t* irun = ibase + (cfirst + (int64_t)j * g.d) * isC;
        const uint32_t nwords = (rows_of(j) * nln * E) >> 2;
#pragma unroll
        for (int k = 0; k < N; ++k) {
          const uint32_t i = tid + (uint32_t)k * kThreads;
          ld_word_pair(irun, i, i < nwords, &lo[k], &hi[k]);
        }
      };
      load(0);
      for (int j = 0; j < nsub; ++j) {
        const uint32_t ncn = rows_of(j), nel = ncn * nln, run = nel * E, nwords = run >> 2;
        const uint8_t* irun = ibase + (cfirst + (int64_t)j * g.d) * isC;
#pragma unroll
        for (int k = 0; k < N; ++k) {
          const uint32_t i = tid + (uint32_t)k * kThreads;
          if (i < nwords) *reinterpret_cast<uint32_t*>(smem + swz(i << 2)) = join_word_pair(irun, lo[k], hi[k]);
        }
        if (tid < (run & 3u)) smem[swz((nwords << 2) + tid)] = irun[(nwords << 2) + tid];
        __syncthreads();
        if (j + 1 < nsub) load(j + 1);
        uint8_t* trun = tbase + (cfirst + (int64_t)j * g.d) * ts_row;
        Walk w;
        w.start(row_order ? nln : ncn, tid);
#pragma unroll
        for (int k = 0; k < NE; ++k) {
          if (tid + (uint32_t)k * kThreads < nel)
            *reinterpret_cast<T*>(trun + (int64_t)w.fast * E + (int64_t)w.slow * ts_slow) = *reinterpret_cast<const T*>(smem + staged_at(w));
          w.next();
        }
        __syncthreads();
      }
    }
    return;
  }

  // ---- wide rows
  const int64_t c0 = (int64_t)(in_batch / g.b) * kTransCols;
  const int64_t lfirst = (int64_t)(in_batch % g.b) * (TL * kTransSub);
  const int nsub = (int)min((int64_t)kTransSub, (nL - lfirst + TL - 1) / TL);
  const int nc = (int)min((int64_t)kTransCols, nC - c0);  // image rows of this tile
  const unsigned tx = tid & 31u, ty = tid >> 5;
  constexpr int NW = (int)kThreads / 32;
  auto elems_of = [&](int j) { return (int)min((int64_t)TL, nL - (lfirst + (int64_t)j * TL)); };
  uint8_t* tcol = tbase + (c0 + tx) * (int64_t)E + lfirst * tsL;  // this thread's column on the tensor side
  if (DIR == MLF_PACK) {
    constexpr int N = G::kPerThread;
    T v[N];
    auto load = [&](int j) {
      const int nl = elems_of(j);
      const uint8_t* col = tcol + (int64_t)j * TL * tsL;
#pragma unroll
      for (int k = 0; k < N; ++k) {
        const int l = (int)ty + k * NW;
        v[k] = ((int)tx < nc && l < nl) ? __ldg(reinterpret_cast<const T*>(col + l * tsL)) : T(0);
      }
    };
    load(0);
    for (int j = 0; j < nsub; ++j) {
      const int nl = elems_of(j);
#pragma unroll
      for (int k = 0; k < N; ++k) {
        const int l = (int)ty + k * NW;
        if ((int)tx < nc && l < nl) *reinterpret_cast<T*>(smem + tx * ROW + l * E) = v[k];
      }
      __syncthreads();
      if (j + 1 < nsub) load(j + 1);
      uint8_t* irow = ibase + c0 * isC + (lfirst + (int64_t)j * TL) * E;
      for (int r = (int)ty; r < nc; r += NW) {
        const uint32_t at = (uint32_t)r * ROW;
        mlf::drain_slot(irow + r * isC, smem + (at & ~15u), at & 15u, (uint32_t)nl * E, tx, 32);
      }
      __syncthreads();
    }
  } else {
    constexpr int N = G::kPasses;
    uint32_t lo[N], hi[N];
    const uint32_t w = tid % G::kWordsPerRow, rsub = tid / G::kWordsPerRow;
    auto load = [&](int j) {
      const uint32_t nwords = ((uint32_t)elems_of(j) * E) >> 2;
      const uint8_t* irow = ibase + c0 * isC + (lfirst + (int64_t)j * TL) * E;
#pragma unroll
      for (int k = 0; k < N; ++k) {
        const uint32_t r = rsub + (uint32_t)k * G::kRowsPerPass;
        ld_word_pair(irow + r * isC, w, r < (uint32_t)nc && w < nwords, &lo[k], &hi[k]);
      }
    };
    load(0);
    for (int j = 0; j < nsub; ++j) {
      const int nl = elems_of(j);
      const uint32_t row_len = (uint32_t)nl * E, nwords = row_len >> 2;
      const uint8_t* irow = ibase + c0 * isC + (lfirst + (int64_t)j * TL) * E;
#pragma unroll
      for (int k = 0; k < N; ++k) {
        const uint32_t r = rsub + (uint32_t)k * G::kRowsPerPass;
        if (r < (uint32_t)nc && w < nwords)
          *reinterpret_cast<uint32_t*>(smem + r * ROW + w * 4u) = join_word_pair(irow + r * isC, lo[k], hi[k]);
      }
      const uint32_t tail = row_len & 3u;  // bytes after the last whole word of each row
      if (tail != 0 && tid < (unsigned)nc * tail) {
        const uint32_t r = tid / tail, b = (nwords << 2) + tid % tail;
        smem[r * ROW + b] = irow[r * isC + b];
      }
      __syncthreads();
      if (j + 1 < nsub) load(j + 1);
      uint8_t* col = tcol + (int64_t)j * TL * tsL;
#pragma unroll
      for (int k = 0; k < G::kPerThread; ++k) {
        const int l = (int)ty + k * NW;
        if ((int)tx < nc && l < nl) *reinterpret_cast<T*>(col + l * tsL) = *reinterpret_cast<const T*>(smem + tx * ROW + l * E);
      }
      __syncthreads();
    }
  }
}

template <typename T, int DIR>
__device__ void generic_tile(const Seg& g, uint32_t local, uint8_t* image) {
  const uint64_t first = (uint64_t)local * kGenericTile;
  const uint64_t last = min(first + kGenericTile, g.a);
  const bool ial = g.image_aligned != 0;
  for (uint64_t e = first + threadIdx.x; e < last; e += blockDim.x) {
    uint64_t r = e;
    int64_t toff = 0, ioff = 0;
    for (int d = (int)g.ndim - 1; d >= 0; --d) {
      const int64_t idx = (int64_t)(r % (uint64_t)g.shape[d]);
      r /= (uint64_t)g.shape[d];
      toff += idx * g.tstride[d];
      ioff += idx * g.istride[d];
    }
    uint8_t* tp = reinterpret_cast<uint8_t*>(g.tensor) + toff;
    uint8_t* ip = image + g.image_off + ioff;
    if (DIR == MLF_PACK)
      store_elem<T>(ip, *reinterpret_cast<const T*>(tp), ial);
    else
      *reinterpret_cast<T*>(tp) = load_elem<T>(ip, ial);
  }
}

template <int DIR>
__device__ __forceinline__ void rows_tile(const Seg& g, uint32_t local, uint8_t* image) {
  const int outer = (int)g.ndim - 1;
  if (g.b == 0) {
    // long rows: this tile is one chunk of one row, moved by the whole CTA
    uint64_t row = local / g.c;
    const uint64_t chunk = local % g.c;
    int64_t toff = 0, ioff = 0;
    for (int d = outer - 1; d >= 0; --d) {
      const int64_t idx = (int64_t)(row % (uint64_t)g.shape[d]);
      row /= (uint64_t)g.shape[d];
      toff += idx * g.tstride[d];
      ioff += idx * g.istride[d];
    }
    const uint64_t off = chunk * kTileBytes;
    const uint64_t len = min(kTileBytes, g.a - off);
    uint8_t* tp = reinterpret_cast<uint8_t*>(g.tensor) + toff + off;
    uint8_t* ip = image + g.image_off + ioff + off;
    if (DIR == MLF_PACK)
      mlf::copy_bytes(ip, tp, len, threadIdx.x, blockDim.x);
    else
      mlf::copy_bytes(tp, ip, len, threadIdx.x, blockDim.x);
    return;
  }
  // short rows: a warp per row
  uint64_t nrows = 1;
  for (int d = 0; d < outer; ++d) nrows *= (uint64_t)g.shape[d];
  const uint64_t r0 = (uint64_t)local * g.b;
  const uint64_t r1 = min(r0 + g.b, nrows);
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (uint64_t r = r0 + warp; r < r1; r += nwarps) {
    uint64_t row = r;
    int64_t toff = 0, ioff = 0;
    for (int d = outer - 1; d >= 0; --d) {
      const int64_t idx = (int64_t)(row % (uint64_t)g.shape[d]);
      row /= (uint64_t)g.shape[d];
      toff += idx * g.tstride[d];
      ioff += idx * g.istride[d];
    }
    uint8_t* tp = reinterpret_cast<uint8_t*>(g.tensor) + toff;
    uint8_t* ip = image + g.image_off + ioff;
    if (DIR == MLF_PACK)
      mlf::copy_bytes(ip, tp, g.a, lane, 32);
    else
      mlf::copy_bytes(tp, ip, g.a, lane, 32);
  }
}

template <int DIR>
__global__ void __launch_bounds__(kThreads) mlf_plan_kernel(const Seg* __restrict__ segs,
                                                            const uint32_t* __restrict__ tile_begin, uint32_t nseg,
                                                            uint32_t ntiles, uint8_t* __restrict__ image) {
  __shared__ __align__(16) uint8_t smem[kTransSmemBytes];
  __shared__ Seg g;
  uint32_t cached = 0xffffffffu;
  for (uint32_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    uint32_t lo = 0, hi = nseg;
    while (hi - lo > 1) {
      const uint32_t mid = (lo + hi) >> 1;
      if (tile_begin[mid] <= tile)
        lo = mid;
      else
        hi = mid;
    }
    if (lo != cached) {  // uniform: every thread ran the same search
      __syncthreads();
      const uint32_t* src = reinterpret_cast<const uint32_t*>(segs + lo);
      uint32_t* dst = reinterpret_cast<uint32_t*>(&g);
      for (uint32_t w = threadIdx.x; w < sizeof(Seg) / 4; w += blockDim.x) dst[w] = src[w];
      __syncthreads();
      cached = lo;
    }
    const uint32_t local = tile - tile_begin[lo];
    switch (g.kind) {
      case kFlat: {
        // tiles are cut on 64 KiB boundaries of the DESTINATION address space, so that only the
        // first and last tile of a segment have ragged edges
        const uint64_t lo_edge = (uint64_t)local * kTileBytes;
        const uint64_t off = lo_edge > g.b ? lo_edge - g.b : 0;
        const uint64_t len = min(lo_edge + kTileBytes - g.b, g.a) - off;
        uint8_t* tp = reinterpret_cast<uint8_t*>(g.tensor) + off;
        uint8_t* ip = image + g.image_off + off;
        if (DIR == MLF_PACK)
          mlf::copy_bytes(ip, tp, len, threadIdx.x, blockDim.x);
        else
          mlf::copy_bytes(tp, ip, len, threadIdx.x, blockDim.x);
        break;
      }
      case kRows:
        rows_tile<DIR>(g, local, image);
        break;
      case kTranspose:
        switch (g.esize) {
          case 1: transpose_tile<uint8_t, DIR>(g, local, image, smem); break;
          case 2: transpose_tile<uint16_t, DIR>(g, local, image, smem); break;
          case 4: transpose_tile<uint32_t, DIR>(g, local, image, smem); break;
          default: transpose_tile<uint64_t, DIR>(g, local, image, smem); break;
        }
        break;
      default:
        switch (g.esize) {
          case 1: generic_tile<uint8_t, DIR>(g, local, image); break;
          case 2: generic_tile<uint16_t, DIR>(g, local, image); break;
          case 4: generic_tile<uint32_t, DIR>(g, local, image); break;
          default: generic_tile<uint64_t, DIR>(g, local, image); break;
        }
        break;
    }
  }
}

// A tile that is not one linear run: short rows, transposed sub-tiles, or single elements.
#ifndef MLF_STAGED_ATTR
#define MLF_STAGED_ATTR
#endif
template <int DIR>
__device__ MLF_STAGED_ATTR void staged_tile(const Seg& g, uint32_t local, uint8_t* image, uint8_t* tsmem, uint8_t* vsmem) {
  if (g.kind == kRows) {
    rows_tile<DIR>(g, local, image);
  } else if (DIR == MLF_PACK && g.kind == kTranspose && g.d == 0 && g.reserved == 4) {
    if (g.esize == 2)
      transpose_tile_m<2, false>(g, local, image, vsmem, tsmem);
    else
      transpose_tile_m<4, false>(g, local, image, vsmem, tsmem);
  } else if (DIR == MLF_PACK && g.kind == kTranspose && g.d == 0 && g.reserved == 6) {
    if (g.esize == 2)
      transpose_tile_m<2, true>(g, local, image, vsmem, tsmem);
    else
      transpose_tile_m<4, true>(g, local, image, vsmem, tsmem);
  } else if (DIR == MLF_PACK && g.kind == kTranspose && g.d == 0 && g.reserved == 5) {
    transpose_tile_ms<2>(g, local, image, vsmem, tsmem);
  } else if (DIR == MLF_PACK && g.kind == kTranspose && g.d == 0 && g.reserved == 2) {
    // wide rows in vector form: staged in `vsmem` (kTransVSmemBytes)
    switch (g.esize) {
      case 1: transpose_tile_v<uint8_t, MLF_PACK>(g, local, image, vsmem); break;
      case 2: transpose_tile_v<uint16_t, MLF_PACK>(g, local, image, vsmem); break;
      case 4: transpose_tile_v<uint32_t, MLF_PACK>(g, local, image, vsmem); break;
      default: transpose_tile_v<uint64_t, MLF_PACK>(g, local, image, vsmem); break;
    }
  } else if (DIR == MLF_PACK && g.kind == kTranspose && g.d != 0 && g.reserved == 7) {
    // narrow transposed rows, pipelined: stages and staging halves in `vsmem` (the idle ring)
    switch (g.esize) {
      case 1: transpose_narrow_async<uint8_t>(g, local, image, vsmem); break;
      case 2: transpose_narrow_async<uint16_t>(g, local, image, vsmem); break;
      case 4: transpose_narrow_async<uint32_t>(g, local, image, vsmem); break;
      default: transpose_narrow_async<uint64_t>(g, local, image, vsmem); break;
    }
  } else if (g.kind == kTranspose) {
    switch (g.esize) {
      case 1: transpose_tile<uint8_t, DIR>(g, local, image, tsmem); break;
      case 2: transpose_tile<uint16_t, DIR>(g, local, image, tsmem); break;
      case 4: transpose_tile<uint32_t, DIR>(g, local, image, tsmem); break;
      default: transpose_tile<uint64_t, DIR>(g, local, image, tsmem); break;
    }
  } else {
    switch (g.esize) {
      case 1: generic_tile<uint8_t, DIR>(g, local, image); break;
      case 2: generic_tile<uint16_t, DIR>(g, local, image); break;
      case 4: generic_tile<uint32_t, DIR>(g, local, image); break;
      default: generic_tile<uint64_t, DIR>(g, local, image); break;
    }
  }
}

// ---- bulk-copy staged variant -------------------------------------------------------------
// Same tiles, same bytes. Linear tiles (FLAT, and chunks of long ROWS) stream through the
// shared-memory ring of bulk_pipeline.cuh; the other kinds run exactly as in mlf_plan_kernel.

// One tile of the streaming phase: a single contiguous run (rows == 0), or `rows` whole short rows
// of segment `seg` starting at flattened row number `first_row`, each `len` bytes.
struct LinearTile {
  const uint8_t* src;
  uint8_t* dst;
  uint64_t len;
  uint32_t nstage;
  uint32_t rows;            // 0: one run; otherwise the number of rows in this tile
  uint32_t rows_per_stage;  // short rows: how many share one ring slot
  uint32_t pitch;           // short rows: bytes between rows inside a slot
  uint64_t first_row;
  const Seg* seg;
};

constexpr uint32_t kMaxStageRows = 32;  // one producer lane per row

// Slot pitch of short rows: room for the row behind a source shift of up to 15 bytes, rounded to
// whole granules, plus the granule the shifted drain reads ahead.
__device__ __host__ __forceinline__ uint32_t short_row_pitch(uint32_t row_bytes) { return ((row_bytes + 30u) & ~15u) + 16u; }

// Span of tile `local` of segment g if the tile belongs to the streaming phase.
template <int DIR>
__device__ __forceinline__ bool linear_span(const Seg& g, uint32_t local, uint8_t* image, LinearTile* out) {
  uint64_t toff, ioff, len;
  out->rows = 0;
  if (g.kind == kFlat) {
    const uint64_t lo_edge = (uint64_t)local * kTileBytes;
    const uint64_t off = lo_edge > g.b ? lo_edge - g.b : 0;
    len = min(lo_edge + kTileBytes - g.b, g.a) - off;
    toff = off;
    ioff = off;
  } else if (g.kind == kRows && g.b == 0) {
    uint64_t row = local / g.c;
    const uint64_t chunk = local % g.c;
    int64_t t = 0, i = 0;
    for (int d = (int)g.ndim - 2; d >= 0; --d) {
      const int64_t idx = (int64_t)(row % (uint64_t)g.shape[d]);
      row /= (uint64_t)g.shape[d];
      t += idx * g.tstride[d];
      i += idx * g.istride[d];
    }
    const uint64_t off = chunk * kTileBytes;
    len = min(kTileBytes, g.a - off);
    toff = (uint64_t)t + off;
    ioff = (uint64_t)i + off;
  } else if (g.kind == kRows) {
    // short rows: g.b of them per tile, several per ring slot
    uint64_t nrows = 1;
    for (int d = 0; d < (int)g.ndim - 1; ++d) nrows *= (uint64_t)g.shape[d];
    const uint64_t r0 = (uint64_t)local * g.b;
    out->first_row = r0;
    out->rows = (uint32_t)min((uint64_t)g.b, nrows - r0);
    out->pitch = short_row_pitch((uint32_t)g.a);
    out->rows_per_stage = min(kMaxStageRows, mlf::kStageBytes / out->pitch);
    out->len = g.a;
    out->nstage = (out->rows + out->rows_per_stage - 1) / out->rows_per_stage;
    out->seg = &g;
    out->src = nullptr;
    out->dst = nullptr;
    return true;
  } else {
    return false;
  }
  uint8_t* tp = reinterpret_cast<uint8_t*>(g.tensor) + toff;
  uint8_t* ip = image + g.image_off + ioff;
  out->src = DIR == MLF_PACK ? tp : ip;
  out->dst = DIR == MLF_PACK ? ip : tp;
  out->len = len;
  out->nstage = (uint32_t)((len + mlf::kStageBytes - 1) / mlf::kStageBytes);
  return true;
}

__device__ __forceinline__ uint32_t find_segment(const uint32_t* __restrict__ tile_begin, uint32_t nseg, uint32_t tile) {
  uint32_t lo = 0, hi = nseg;
  while (hi - lo > 1) {
    const uint32_t mid = (lo + hi) >> 1;
    if (tile_begin[mid] <= tile)
      lo = mid;
    else
      hi = mid;
  }
  return lo;
}

// The plan tables list the segments made of linear tiles first: tiles [0, nlinear) are linear runs,
// tiles [nlinear, ntiles) are staged tiles (short rows, transposed sub-tiles, single elements).
//
// Streaming phase over this CTA's linear tiles. One elected thread walks the tiles, issues the
// bulk loads and publishes, per ring slot, where the slot's bytes go; the other threads never look
// at the plan tables: they wait for a slot, read its destination from shared memory and drain it.
// A slot whose published length is 0 ends the phase. Returns false if a bounded wait ran out
// (status recorded, outstanding copies awaited): the CTA must then return.
struct SlotMeta {
  uint8_t* dst;    // one run: destination of the slot's first payload byte
  uint32_t len;    // payload bytes of the run, or of each row; 0 = no more stages
  uint32_t shift;  // one run: the payload starts this many bytes into the slot (source misalignment)
  uint32_t rows;   // 0: the slot holds one run; otherwise this many short rows, `pitch` bytes apart
  uint32_t pitch;
};

// Shared memory of the streaming phase besides the ring itself.
struct StreamShared {
  uint64_t full[mlf::kStages];  // one mbarrier per slot
  SlotMeta meta[mlf::kStages];
  uint8_t* row_dst[mlf::kStages][kMaxStageRows];  // short rows: where each row of the slot goes
  uint8_t row_shift[mlf::kStages][kMaxStageRows];
  int abort_flag;
};

template <int DIR>
__device__ __forceinline__ bool stream_linear_tiles(const Seg* __restrict__ segs, const uint32_t* __restrict__ tile_begin,
                                                    uint32_t nseg, uint32_t nlinear, uint8_t* __restrict__ image,
                                                    int32_t* __restrict__ status, uint8_t* ring, StreamShared* sh) {
  const unsigned tid = threadIdx.x, lane = tid & 31u;
  // producer state, kept identically by all lanes of warp 0
  uint32_t p_tile = blockIdx.x, p_stage = 0, issued = 0;
  bool p_finished = false;
  LinearTile p_lt;
  p_lt.nstage = 0;
  p_lt.rows = 0;
  auto seek = [&]() {  // loads the span of tile p_tile
    if (p_tile < nlinear) {
      const uint32_t sg = find_segment(tile_begin, nseg, p_tile);
      (void)linear_span<DIR>(segs[sg], p_tile - tile_begin[sg], image, &p_lt);
    }
  };
  // Fills every free slot: slot (issued % kStages) is free once stage (issued - kStages) was drained.
  // Runs on warp 0 with all lanes: lane 0 issues the load of a run, lane r the load of a slot's row r.
  auto top_up = [&](uint32_t consumed) {
    while (issued < consumed + mlf::kStages && !p_finished) {
      const uint32_t slot = issued % mlf::kStages;
      uint8_t* slot_base = ring + (size_t)slot * mlf::kSlotBytes;
      if (p_tile >= nlinear) {
        if (lane == 0) sh->meta[slot].len = 0;
        p_finished = true;
        ++issued;
        break;
      }
      if (p_lt.rows == 0) {
        if (lane == 0) {
          const uint64_t off = (uint64_t)p_stage * mlf::kStageBytes;
          const uint32_t slen = (uint32_t)min((uint64_t)mlf::kStageBytes, p_lt.len - off);
          const uint8_t* src = p_lt.src + off;
          const uint32_t shift = (uint32_t)((uintptr_t)src & 15u);
          const uint32_t bytes = (shift + slen + 15u) & ~15u;
          sh->meta[slot].dst = p_lt.dst + off;
          sh->meta[slot].len = slen;
          sh->meta[slot].shift = shift;
          sh->meta[slot].rows = 0;
          mlf::mbar_expect_tx(&sh->full[slot], bytes);
          mlf::bulk_load(slot_base, src - shift, bytes, &sh->full[slot]);
        }
      } else {
        const Seg& g = *p_lt.seg;
        const uint32_t r_in_tile = p_stage * p_lt.rows_per_stage;
        const uint32_t n = min(p_lt.rows_per_stage, p_lt.rows - r_in_tile);
        const uint8_t* src = nullptr;
        uint32_t shift = 0, bytes = 0;
        if (lane < n) {
          uint64_t row = p_lt.first_row + r_in_tile + lane;
          int64_t t = 0, i = 0;
          for (int d = (int)g.ndim - 2; d >= 0; --d) {
            const int64_t idx = (int64_t)(row % (uint64_t)g.shape[d]);
            row /= (uint64_t)g.shape[d];
            t += idx * g.tstride[d];
            i += idx * g.istride[d];
          }
          uint8_t* tp = reinterpret_cast<uint8_t*>(g.tensor) + t;
          uint8_t* ip = image + g.image_off + i;
          src = DIR == MLF_PACK ? tp : ip;
          shift = (uint32_t)((uintptr_t)src & 15u);
          bytes = (shift + (uint32_t)p_lt.len + 15u) & ~15u;
          sh->row_dst[slot][lane] = DIR == MLF_PACK ? ip : tp;
          sh->row_shift[slot][lane] = (uint8_t)shift;
        }
        uint32_t total = bytes;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        if (lane == 0) {
          sh->meta[slot].dst = nullptr;
          sh->meta[slot].len = (uint32_t)p_lt.len;
          sh->meta[slot].shift = 0;
          sh->meta[slot].rows = n;
          sh->meta[slot].pitch = p_lt.pitch;
          mlf::mbar_expect_tx(&sh->full[slot], total);
        }
        __syncwarp();
        if (lane < n) mlf::bulk_load(slot_base + (size_t)lane * p_lt.pitch, src - shift, bytes, &sh->full[slot]);
      }
      ++issued;
      if (++p_stage == p_lt.nstage) {
        p_stage = 0;
        p_tile += gridDim.x;
        seek();
      }
    }
  };

  if (tid == 0) {
    for (uint32_t k = 0; k < mlf::kStages; ++k) mlf::mbar_init(&sh->full[k], 1);
    mlf::mbar_init_fence();
    sh->abort_flag = 0;
  }
  __syncthreads();
  if (tid < 32) {
    seek();
    top_up(0);
  }
  __syncthreads();  // publishes the first slots' destinations

  uint32_t consumed = 0;
  bool aborted = false;
  for (;;) {
    const uint32_t slot = consumed % mlf::kStages;
    // written by warp 0 at least one barrier ago: stage `consumed` was issued before the barrier
    // that ended stage `consumed - 1` (or before the barrier above)
    const SlotMeta m = sh->meta[slot];
    if (m.len == 0) break;
    const bool ok = mlf::mbar_wait_bounded(&sh->full[slot], (consumed / mlf::kStages) & 1u);
    if (ok) {
      const uint8_t* slot_base = ring + (size_t)slot * mlf::kSlotBytes;
      if (m.rows == 0) {
        mlf::drain_slot(m.dst, slot_base, m.shift, m.len, tid, blockDim.x);
      } else {
        for (uint32_t r = tid >> 5; r < m.rows; r += blockDim.x >> 5)
          mlf::drain_slot(sh->row_dst[slot][r], slot_base + (size_t)r * m.pitch, sh->row_shift[slot][r], m.len, lane, 32);
      }
    } else {
      sh->abort_flag = 1;
    }
    __syncthreads();  // the slot is free again; also publishes abort_flag
    ++consumed;
    if (sh->abort_flag) {
      aborted = true;
      break;
    }
    if (tid < 32) top_up(consumed);  // refills the slot just freed; its destination is published by the next barrier
  }
  if (aborted && tid == 0) {
    atomicCAS(status, 0, MLF_ERR_TIMEOUT);
    // the CTA may not exit while bulk copies still target its shared memory: wait for them too,
    // again with a budget (the end marker, if one was written, took a slot number but no load)
    const uint32_t loads_issued = issued - (p_finished ? 1u : 0u);
    for (uint32_t n = consumed - 1; n < loads_issued; ++n)  // from the stage whose wait ran out
      (void)mlf::mbar_wait_bounded(&sh->full[n % mlf::kStages], (n / mlf::kStages) & 1u);
  }
  return !aborted;
}

// Plans made of linear tiles only (every contiguous state dict): the streaming phase is the kernel.
#ifndef MLF_STREAM_MIN_CTAS
#define MLF_STREAM_MIN_CTAS 3
#endif
template <int DIR>
__global__ void __launch_bounds__(kThreads, MLF_STREAM_MIN_CTAS) mlf_plan_kernel_stream(const Seg* __restrict__ segs,
                                                                   const uint32_t* __restrict__ tile_begin, uint32_t nseg,
                                                                   uint32_t nlinear, uint32_t ntiles, uint8_t* __restrict__ image,
                                                                   int32_t* __restrict__ status) {
  extern __shared__ __align__(128) uint8_t ring[];  // kStages slots of kSlotBytes
  __shared__ __align__(16) StreamShared shared;
  (void)ntiles;
  (void)stream_linear_tiles<DIR>(segs, tile_begin, nseg, nlinear, image, status, ring, &shared);
}

// Plans that also hold staged tiles: the streaming phase over the linear tiles, then this CTA's
// share of the staged tiles, each found in the plan tables by all threads.
template <int DIR>
__global__ void __launch_bounds__(kThreads, 3) mlf_plan_kernel_bulk(const Seg* __restrict__ segs,
                                                                 const uint32_t* __restrict__ tile_begin, uint32_t nseg,
                                                                 uint32_t nlinear, uint32_t ntiles, uint8_t* __restrict__ image,
                                                                 int32_t* __restrict__ status) {
  extern __shared__ __align__(128) uint8_t ring[];  // kStages slots of kSlotBytes
  __shared__ __align__(16) StreamShared shared;
  __shared__ __align__(16) uint8_t tsmem[kTransSmemBytes];
  __shared__ Seg g;
  if (!stream_linear_tiles<DIR>(segs, tile_begin, nseg, nlinear, image, status, ring, &shared)) return;
  const unsigned tid = threadIdx.x;
  uint32_t cached = 0xffffffffu;
  // Staged tiles differ in cost by an order of magnitude (a matrix-form tile moves 128 KiB, a tile
  // of single elements 8 KiB), and the CTAs leave the streaming phase at different times: they are
  // handed out one by one from a counter behind the status word (zeroed by the launch), heaviest
  // segments first (the planner's order), instead of in fixed strides.
  __shared__ uint32_t claimed;
  for (;;) {
    if (tid == 0) claimed = nlinear + atomicAdd(reinterpret_cast<unsigned int*>(status) + 1, 1u);
    __syncthreads();
    const uint32_t tile = claimed;
    if (tile >= ntiles) break;
    const uint32_t sg = find_segment(tile_begin, nseg, tile);
    const uint32_t local = tile - tile_begin[sg];
    __syncthreads();  // everyone has read `claimed` (and is done with the previous tile's segment copy)
    if (sg != cached) {
      const uint32_t* src = reinterpret_cast<const uint32_t*>(segs + sg);
      uint32_t* dst = reinterpret_cast<uint32_t*>(&g);
      for (uint32_t w = tid; w < sizeof(Seg) / 4; w += blockDim.x) dst[w] = src[w];
      __syncthreads();
      cached = sg;
    }
    // the ring of the streaming phase is idle by now: it stages the vector- and matrix-form transposes
    staged_tile<DIR>(g, local, image, tsmem, ring);
  }
}

// Self-test of the bounded wait: a barrier that nothing will ever complete. The wait has to give
// up after `budget_ns` and report it through the status word, like the streaming phase does.
__global__ void mlf_wait_selftest_kernel(uint64_t budget_ns, int32_t* __restrict__ status) {
  __shared__ __align__(8) uint64_t never;
  if (threadIdx.x == 0) {
    mlf::mbar_init(&never, 1);
    mlf::mbar_init_fence();
    if (!mlf::mbar_wait_bounded(&never, 0, budget_ns)) atomicCAS(status, 0, MLF_ERR_TIMEOUT);
  }
}

constexpr size_t kBulkDynSmem = (size_t)mlf::kStages * mlf::kSlotBytes;
static_assert(kTransVSmemBytes <= (int)mlf::kSlotBytes, "the vector-form transpose stages through one ring slot");
static_assert(kTransMStagingOff + TransM<2>::kCols * TransM<2>::kPitch <= (int)kBulkDynSmem &&
                  kTransMStagingOff + TransM<4>::kCols * TransM<4>::kPitch <= (int)kBulkDynSmem,
              "matrix form: two stages and the staging area fit the ring");
static_assert(kNarrowASmemBytes <= (int)kBulkDynSmem, "pipelined narrow rows: stages and staging halves fit the ring");
static_assert(2 * TransM<2>::kCarryBytes <= kTransSmemBytes, "matrix form: carries fit the static staging area");

__global__ void __launch_bounds__(kThreads) mlf_flat_copy_kernel(uint8_t* __restrict__ dst,
                                                                 const uint8_t* __restrict__ src, uint64_t nbytes) {
  const uint64_t mis = (uint64_t)((uintptr_t)dst & 127u);
  const uint64_t ntiles = (mis + nbytes + kTileBytes - 1) / kTileBytes;
  for (uint64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const uint64_t lo_edge = t * kTileBytes;
    const uint64_t off = lo_edge > mis ? lo_edge - mis : 0;
    const uint64_t len = min(lo_edge + kTileBytes - mis, nbytes) - off;
    mlf::copy_bytes(dst + off, src + off, len, threadIdx.x, blockDim.x);
  }
}

// ------------------------------------------------------------------------------------ host

// Grid for a persistent launch of `kernel`: one full wave (SMs x resident CTAs per SM), capped by
// the tile count and by the caller's limit.
template <typename K>
int32_t wave_grid(K kernel, int32_t max_ctas, uint64_t ntiles, uint32_t* grid, size_t dyn_smem = 0) {
  int dev = 0, sms = 0, per_sm = 0;
  MLF_CUDA(cudaGetDevice(&dev));
  MLF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  MLF_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, (int)kThreads, dyn_smem));
  uint64_t g = (uint64_t)sms * (uint64_t)std::max(per_sm, 1);
  if (max_ctas > 0) g = std::min<uint64_t>(g, (uint64_t)max_ctas);
  g = std::max<uint64_t>(1, std::min<uint64_t>(g, ntiles));
  *grid = (uint32_t)g;
  return MLF_OK;
}

// Canonical form of one descriptor: unit dims dropped, mergeable neighbours merged, strides in bytes.
struct Canon {
  int ndim = 0;
  int64_t shape[MLF_MAX_DIMS + 1];
  int64_t ts[MLF_MAX_DIMS + 1];
  int64_t is[MLF_MAX_DIMS + 1];
};

Canon canonicalise(uint32_t esize, const int64_t* shape, const int64_t* ts_elems, const int64_t* is_elems, int ndim) {
  Canon c;
  for (int k = 0; k < ndim; ++k) {
    if (shape[k] == 1) continue;
    const int64_t ts = ts_elems[k] * (int64_t)esize, is = is_elems[k] * (int64_t)esize;
    if (c.ndim > 0 && c.ts[c.ndim - 1] == ts * shape[k] && c.is[c.ndim - 1] == is * shape[k]) {
      c.shape[c.ndim - 1] *= shape[k];
      c.ts[c.ndim - 1] = ts;
      c.is[c.ndim - 1] = is;
    } else {
      c.shape[c.ndim] = shape[k];
      c.ts[c.ndim] = ts;
      c.is[c.ndim] = is;
      ++c.ndim;
    }
  }
  return c;
}

// Kernel variant for plan launches: the bulk-copy staged kernel unless MLF_PLAN_KERNEL=ldg asks for
// the register-staged one (kept for comparison and for mlf_pack_noalloc).
bool use_bulk_kernel() {
  static const bool bulk = []() {
    const char* v = getenv("MLF_PLAN_KERNEL");
    return !(v && std::string(v) == "ldg");
  }();
  return bulk;
}

// Form of the wide transposes in pack plans: MLF_TRANSPOSE_FORM = matrix (default) | vector | async | element.
int wide_transpose_form() {
  static const int form = []() {
    const char* v = getenv("MLF_TRANSPOSE_FORM");
    const std::string want = v ? v : "";
    if (want == "element") return 0;
    if (want == "vector") return 2;
    return 4;
  }();
  return form;
}

// ---- scratch of mlf_pack_noalloc ---------------------------------------------------------
// Segment table, tile index and a status word for the entry point that may not allocate. The
// array lives in every device that loads this library, from load until exit.
constexpr uint32_t kNoAllocMaxSegs = MLF_NOALLOC_MAX_DESCS;
constexpr size_t kNoAllocSegBytes = sizeof(Seg) * kNoAllocMaxSegs;
constexpr size_t kNoAllocTileBytes = sizeof(uint32_t) * (kNoAllocMaxSegs + 1);
constexpr size_t kNoAllocStatusOff = (kNoAllocSegBytes + kNoAllocTileBytes + 255) / 256 * 256;
constexpr size_t kNoAllocScratchBytes = kNoAllocStatusOff + 256;
static __device__ __align__(256) uint8_t g_noalloc_scratch[kNoAllocScratchBytes];

// Device address of g_noalloc_scratch per device, resolved on the first call made with that
// device current. (In host code the array's name is only a handle for the runtime, not an address.)
constexpr int kMaxDevices = 64;
uint8_t* g_noalloc_dev_ptr[kMaxDevices] = {nullptr};
std::mutex g_noalloc_mu;  // guards the pointer table and the host staging arrays below
Seg g_noalloc_host_segs[kNoAllocMaxSegs];
uint32_t g_noalloc_host_tiles[kNoAllocMaxSegs + 1];

// Turns one descriptor into a segment: validation, canonical form, kind and tile count.
// On success *ntile_out is 0 if the descriptor moves nothing (the segment is then unused).
// The cp.async-fed matrix form moves 16- and 32-bit elements whose tensor rows all start on
// boundaries of `align` bytes: 16 (granule copies) or 4 (word copies).
bool matrix_form_eligible(uint32_t esize, uint64_t tensor_ptr, const Canon& c, int cdim, uint32_t align) {
  if ((esize != 2 && esize != 4) || (tensor_ptr & (align - 1))) return false;
  for (int k = 0; k < c.ndim; ++k)
    if (k != cdim && (c.ts[k] & (int64_t)(align - 1))) return false;
  return true;
}

// `wide_form`: tile geometry of TRANSPOSE boxes: 0 element-wise, 2 vector form, 4 matrix form for
// 16- and 32-bit elements (cp.async-fed by granules where every tensor row starts on a 16-byte
// boundary, by words where on a 4-byte boundary, register-fed with a shift elsewhere) and vector
// form for the other element sizes; with 2 and 4 narrow rows take the pipelined form (all but 0
// only exist in the bulk kernels, for the pack direction).
int32_t plan_segment(const mlf_copy_desc& d, uint64_t i, int32_t direction, int wide_form, Seg* seg_out, uint64_t* ntile_out,
                     uint64_t* payload_out, uint64_t* extent_out) {
  *ntile_out = 0;
  *payload_out = 0;
  *extent_out = 0;
  {
    const std::string where = "descriptor " + std::to_string(i);
    if (d.ndim > MLF_MAX_DIMS) return mlf::fail(MLF_ERR_INVALID, where + ": ndim exceeds MLF_MAX_DIMS");
    if (d.elem_size != 1 && d.elem_size != 2 && d.elem_size != 4 && d.elem_size != 8 && d.elem_size != 16)
      return mlf::fail(MLF_ERR_INVALID, where + ": elem_size must be 1, 2, 4, 8 or 16");
    // Shapes and strides come from the caller: every product and sum below is checked, so that a
    // wrapped extent can never slip under the image-capacity guard of the launch.
    uint64_t numel = 1;
    uint64_t span = 0;   // highest element index touched on the image side
    uint64_t tspan = 0;  // the same on the tensor side
    bool empty = false, overflow = false;
    for (uint32_t k = 0; k < d.ndim; ++k) {
      if (d.shape[k] < 0 || d.tensor_stride[k] < 0 || d.image_stride[k] < 0)
        return mlf::fail(MLF_ERR_INVALID, where + ": negative extent or stride");
      if (d.shape[k] == 0) empty = true;
    }
    if (empty) return MLF_OK;  // nothing to move; the format stores no payload for it either
    for (uint32_t k = 0; k < d.ndim; ++k) {
      uint64_t step = 0;
      overflow |= __builtin_mul_overflow(numel, (uint64_t)d.shape[k], &numel);
      overflow |= __builtin_mul_overflow((uint64_t)(d.shape[k] - 1), (uint64_t)d.image_stride[k], &step);
      overflow |= __builtin_add_overflow(span, step, &span);
      overflow |= __builtin_mul_overflow((uint64_t)(d.shape[k] - 1), (uint64_t)d.tensor_stride[k], &step);
      overflow |= __builtin_add_overflow(tspan, step, &tspan);
    }
    if (d.tensor_ptr == 0) return mlf::fail(MLF_ERR_INVALID, where + ": null tensor pointer");
    uint64_t payload = 0, extent = 0, tensor_end = 0;
    overflow |= __builtin_mul_overflow(numel, (uint64_t)d.elem_size, &payload);
    overflow |= __builtin_add_overflow(span, (uint64_t)1, &extent);
    overflow |= __builtin_mul_overflow(extent, (uint64_t)d.elem_size, &extent);
    overflow |= __builtin_add_overflow(extent, d.image_off, &extent);
    overflow |= __builtin_add_overflow(tspan, (uint64_t)1, &tensor_end);
    overflow |= __builtin_mul_overflow(tensor_end, (uint64_t)d.elem_size, &tensor_end);
    overflow |= __builtin_add_overflow(tensor_end, d.tensor_ptr, &tensor_end);
    // byte strides are kept as int64 further down; 2^62 leaves room for the x2 of 16-byte elements
    overflow |= payload >> 62 || extent >> 62 || (tensor_end - d.tensor_ptr) >> 62;
    if (overflow)
      return mlf::fail(MLF_ERR_INVALID, where + ": shape and strides overflow 64-bit byte arithmetic");
    *payload_out = payload;
    *extent_out = extent;

    // 16-byte elements are moved as pairs of 8-byte halves (an extra innermost dimension of 2)
    int64_t shp[MLF_MAX_DIMS + 1], ts[MLF_MAX_DIMS + 1], is[MLF_MAX_DIMS + 1];
    int nd = (int)d.ndim;
    uint32_t esize = d.elem_size;
    for (int k = 0; k < nd; ++k) {
      shp[k] = d.shape[k];
      ts[k] = d.tensor_stride[k];
      is[k] = d.image_stride[k];
    }
    if (esize == 16) {
      for (int k = 0; k < nd; ++k) {
        ts[k] *= 2;
        is[k] *= 2;
      }
      shp[nd] = 2;
      ts[nd] = 1;
      is[nd] = 1;
      ++nd;
      esize = 8;
    }
    const Canon c = canonicalise(esize, shp, ts, is, nd);
    if (c.ndim > MLF_MAX_DIMS)
      return mlf::fail(MLF_ERR_INVALID, where + ": too many dimensions after splitting 16-byte elements");

    Seg& g = *seg_out;
    memset(&g, 0, sizeof(g));
    g.tensor = d.tensor_ptr;
    g.image_off = d.image_off;
    g.esize = esize;
    g.ndim = (uint32_t)c.ndim;
    bool aligned = (d.image_off % esize) == 0;
    for (int k = 0; k < c.ndim; ++k) {
      g.shape[k] = c.shape[k];
      g.tstride[k] = c.ts[k];
      g.istride[k] = c.is[k];
      if (c.is[k] % esize) aligned = false;
    }
    g.image_aligned = aligned ? 1u : 0u;
    if ((d.tensor_ptr % esize) != 0)
      return mlf::fail(MLF_ERR_INVALID, where + ": tensor pointer is not aligned to its element size");

    const int last = c.ndim - 1;
    const bool inner_contig = c.ndim == 0 || (c.ts[last] == (int64_t)esize && c.is[last] == (int64_t)esize);
    uint64_t ntile = 0;
    if (c.ndim == 0 || (c.ndim == 1 && inner_contig)) {
      g.kind = kFlat;
      g.a = numel * d.elem_size;
      // the image base is at least 128-byte aligned in practice (HBM allocations, page-aligned
      // mappings); if it is not, only the tile edges move, never the bytes
      g.b = (uint32_t)((direction == MLF_PACK ? d.image_off : d.tensor_ptr) & 127u);
      ntile = (g.b + g.a + kTileBytes - 1) / kTileBytes;
    } else if (inner_contig && c.ndim >= 2 && (uint64_t)c.shape[last] * esize < trans_row_bytes(esize) &&
               (uint64_t)c.is[last - 1] == (uint64_t)c.shape[last] * esize) {
      // short rows that lie back to back in the image: staged like narrow TRANSPOSE rows, walked in row order
      g.kind = kTranspose;
      g.c = (uint32_t)(last - 1);
      g.reserved = 1;
      const uint64_t row_bytes = (uint64_t)c.shape[last] * esize;
      g.d = (uint32_t)std::max<uint64_t>(1, (uint64_t)trans_narrow_bytes(esize) / row_bytes);
      const uint64_t rows_per_tile = (uint64_t)g.d * kTransSub;
      g.a = ((uint64_t)c.shape[last - 1] + rows_per_tile - 1) / rows_per_tile;
      g.b = 1;
      uint64_t batch = 1;
      for (int k = 0; k < last - 1; ++k) batch *= (uint64_t)c.shape[k];
      ntile = batch * g.a;
      if (g.a > 0xffffffffull) return mlf::fail(MLF_ERR_TOO_LARGE, where + ": box too large");
    } else if (inner_contig) {
      g.kind = kRows;
      g.a = (uint64_t)c.shape[last] * esize;
      uint64_t nrows = 1;
      for (int k = 0; k < last; ++k) nrows *= (uint64_t)c.shape[k];
      if (g.a >= kRowSplitBytes) {
        g.b = 0;
        g.c = (uint32_t)((g.a + kTileBytes - 1) / kTileBytes);
        ntile = nrows * g.c;
      } else {
        g.b = (uint32_t)std::min<uint64_t>(kRowsPerTileMax, std::max<uint64_t>(1, kTileBytes / g.a));
        ntile = (nrows + g.b - 1) / g.b;
      }
    } else {
      int cdim = -1;
      if (c.is[last] == (int64_t)esize)
        for (int k = 0; k < last; ++k)
          if (c.ts[k] == (int64_t)esize) cdim = k;
      if (cdim >= 0) {
        g.kind = kTranspose;
        g.c = (uint32_t)cdim;
        const uint64_t row_cap = trans_row_bytes(esize);
        const uint64_t per_row = row_cap / esize;
        const uint64_t row_bytes = (uint64_t)c.shape[last] * esize;
        uint64_t tc, tl;
        // The pipelined narrow form takes rows of up to 127 elements (its bound on granules per
        // sub-tile): 32- and 64-bit rows too short to fill one 128-row stage of the wide forms.
        const bool narrow = row_bytes < row_cap || (wide_form != 0 && esize >= 4 && c.shape[last] <= kNarrowAMaxRow);
        if (narrow && (uint64_t)c.is[cdim] == row_bytes) {
          // short image rows lying back to back: a sub-tile is as many whole rows as fit the staging area
          g.d = (uint32_t)std::max<uint64_t>(1, (uint64_t)trans_narrow_bytes(esize) / row_bytes);
          if (wide_form != 0) g.reserved = 7;  // pack plans of the bulk kernels: pipelined form, longer tiles
          const uint64_t rows_per_tile = (uint64_t)g.d * (wide_form != 0 ? kNarrowASub : kTransSub);
          tc = ((uint64_t)c.shape[cdim] + rows_per_tile - 1) / rows_per_tile;
          tl = 1;
        } else if (wide_form == 4 && matrix_form_eligible(esize, d.tensor_ptr, c, cdim, 4)) {
          const uint64_t cols = trans_m_cols(esize);
          g.reserved = matrix_form_eligible(esize, d.tensor_ptr, c, cdim, 16) ? 4 : 6;  // granule-fed or word-fed
          tc = ((uint64_t)c.shape[cdim] + cols - 1) / cols;
          tl = ((uint64_t)c.shape[last] + (uint64_t)kTransML * kTransMSub - 1) / ((uint64_t)kTransML * kTransMSub);
        } else if (wide_form == 4 && esize == 2) {
          // 16-bit rows on 2-byte boundaries (wider elements are at least word-aligned): matrix form behind a register-side shift
          const uint64_t cols = trans_ms_cols(esize);
          tc = ((uint64_t)c.shape[cdim] + cols - 1) / cols;
          tl = ((uint64_t)c.shape[last] + (uint64_t)kTransML * kTransMSub - 1) / ((uint64_t)kTransML * kTransMSub);
          g.reserved = 5;
        } else if (wide_form == 2 || wide_form == 4) {
          const uint64_t cols = trans_v_cols(esize);
          tc = ((uint64_t)c.shape[cdim] + cols - 1) / cols;
          tl = ((uint64_t)c.shape[last] + (uint64_t)kTransVL * kTransSub - 1) / ((uint64_t)kTransVL * kTransSub);
          g.reserved = 2;
        } else {
          tc = ((uint64_t)c.shape[cdim] + kTransCols - 1) / kTransCols;
          tl = ((uint64_t)c.shape[last] + per_row * kTransSub - 1) / (per_row * kTransSub);
        }
        g.b = (uint32_t)tl;
        g.a = tc * tl;
        uint64_t batch = 1;
        for (int k = 0; k < last; ++k)
          if (k != cdim) batch *= (uint64_t)c.shape[k];
        ntile = batch * g.a;
        if (g.a > 0xffffffffull) return mlf::fail(MLF_ERR_TOO_LARGE, where + ": transposed box too large");
      } else {
        g.kind = kGeneric;
        g.a = numel * (d.elem_size / esize);
        ntile = (g.a + kGenericTile - 1) / kGenericTile;
      }
    }
    *ntile_out = ntile;
  }
  return MLF_OK;
}

}  // namespace

struct mlf_plan {
  int direction = MLF_PACK;
  int device = 0;
  uint32_t nseg = 0;
  uint32_t ntiles = 0;
  uint64_t extent = 0;
  uint64_t payload = 0;
  uint32_t nlinear = 0;  // tiles [0, nlinear) are linear runs, the rest are staged tiles
  Seg* d_segs = nullptr;
  uint32_t* d_tile_begin = nullptr;
  int32_t* d_status = nullptr;
};

extern "C" {

int32_t mlf_plan_create(const mlf_copy_desc* descs, uint64_t n, int32_t direction, mlf_plan** out) {
  if (!out) return mlf::fail(MLF_ERR_INVALID, "mlf_plan_create: null out");
  *out = nullptr;
  if (n > 0 && !descs) return mlf::fail(MLF_ERR_INVALID, "mlf_plan_create: null descriptors");
  if (direction != MLF_PACK && direction != MLF_UNPACK)
    return mlf::fail(MLF_ERR_INVALID, "mlf_plan_create: direction must be MLF_PACK or MLF_UNPACK");

  // Segments in table order: those made of linear tiles first, so that tiles [0, nlinear) are the
  // linear ones (a segment carries its own addresses, so the table order is free).
  // the vector-form transposes stage through the ring's shared memory, which only the bulk kernels have
  // (pack only: scattering into tensor granules measured slower than the element-wise form)
  const int wide_form = direction == MLF_PACK && use_bulk_kernel() ? wide_transpose_form() : 0;
  std::vector<Seg> linear_segs, staged_segs;
  std::vector<uint64_t> linear_tiles, staged_tiles, staged_payload;
  uint64_t tiles = 0, extent = 0, payload = 0;

  for (uint64_t i = 0; i < n; ++i) {
    Seg g;
    uint64_t ntile = 0, seg_payload = 0, seg_extent = 0;
    const int32_t rc = plan_segment(descs[i], i, direction, wide_form, &g, &ntile, &seg_payload, &seg_extent);
    if (rc != MLF_OK) return rc;
    if (ntile == 0) continue;
    payload += seg_payload;
    extent = std::max(extent, seg_extent);
    if (tiles + ntile > 0xfffffff0ull) return mlf::fail(MLF_ERR_TOO_LARGE, "plan has too many tiles");
    tiles += ntile;
    const bool linear = g.kind == kFlat || g.kind == kRows;  // everything the streaming phase moves
    (linear ? linear_segs : staged_segs).push_back(g);
    (linear ? linear_tiles : staged_tiles).push_back(ntile);
    if (!linear) staged_payload.push_back(seg_payload);
  }
  // staged segments in order of bytes per tile, heaviest first: the kernel hands staged tiles out
  // dynamically, and starting with the big ones leaves the small ones to even out the finish
  {
    std::vector<size_t> order(staged_segs.size());
    for (size_t k = 0; k < order.size(); ++k) order[k] = k;
    std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) {
      return staged_payload[a] * staged_tiles[b] > staged_payload[b] * staged_tiles[a];  // payload / tiles, without dividing
    });
    std::vector<Seg> sorted_segs;
    std::vector<uint64_t> sorted_tiles;
    for (size_t k : order) {
      sorted_segs.push_back(staged_segs[k]);
      sorted_tiles.push_back(staged_tiles[k]);
    }
    staged_segs.swap(sorted_segs);
    staged_tiles.swap(sorted_tiles);
  }
  std::vector<Seg> segs(linear_segs);
  segs.insert(segs.end(), staged_segs.begin(), staged_segs.end());
  std::vector<uint32_t> tile_begin;
  tile_begin.reserve(segs.size() + 1);
  uint64_t at = 0, nlinear = 0;
  for (uint64_t ntile : linear_tiles) {
    tile_begin.push_back((uint32_t)at);
    at += ntile;
  }
  nlinear = at;
  for (uint64_t ntile : staged_tiles) {
    tile_begin.push_back((uint32_t)at);
    at += ntile;
  }
  tile_begin.push_back((uint32_t)at);

  mlf_plan* p = new mlf_plan();
  p->nlinear = (uint32_t)nlinear;
  p->direction = direction;
  p->nseg = (uint32_t)segs.size();
  p->ntiles = (uint32_t)tiles;
  p->extent = extent;
  p->payload = payload;
  cudaError_t e = cudaGetDevice(&p->device);
  if (e == cudaSuccess && p->nseg > 0) {
    e = cudaMalloc(&p->d_segs, segs.size() * sizeof(Seg));
    if (e == cudaSuccess) e = cudaMalloc(&p->d_tile_begin, tile_begin.size() * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMalloc(&p->d_status, 2 * sizeof(int32_t));  // status word, staged-tile counter
    if (e == cudaSuccess) e = cudaMemcpy(p->d_segs, segs.data(), segs.size() * sizeof(Seg), cudaMemcpyHostToDevice);
    if (e == cudaSuccess)
      e = cudaMemcpy(p->d_tile_begin, tile_begin.data(), tile_begin.size() * sizeof(uint32_t), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemset(p->d_status, 0, 2 * sizeof(int32_t));
  }
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    mlf_plan_destroy(p);
    return mlf::cuda_fail(e, "uploading the plan tables");
  }
  *out = p;
  return MLF_OK;
}

void mlf_plan_destroy(mlf_plan* p) {
  if (!p) return;
  if (p->d_segs) cudaFree(p->d_segs);
  if (p->d_tile_begin) cudaFree(p->d_tile_begin);
  if (p->d_status) cudaFree(p->d_status);
  delete p;
}

uint64_t mlf_plan_image_extent(const mlf_plan* p) { return p ? p->extent : 0; }
uint64_t mlf_plan_payload_bytes(const mlf_plan* p) { return p ? p->payload : 0; }
uint64_t mlf_plan_num_tiles(const mlf_plan* p) { return p ? p->ntiles : 0; }

int32_t mlf_plan_launch(mlf_plan* p, void* image_base, uint64_t image_capacity, void* stream, int32_t max_ctas) {
  if (!p) return mlf::fail(MLF_ERR_INVALID, "mlf_plan_launch: null plan");
  if (p->extent > image_capacity)
    return mlf::fail(MLF_ERR_BOUNDS, "plan touches " + std::to_string(p->extent) + " image bytes but only " +
                                         std::to_string(image_capacity) + " are available");
  if (p->ntiles == 0) return MLF_OK;
  if (!image_base) return mlf::fail(MLF_ERR_INVALID, "mlf_plan_launch: null image");
  uint32_t grid = 1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* image = static_cast<uint8_t*>(image_base);
  if (use_bulk_kernel()) {
    using BulkKernel = void (*)(const Seg*, const uint32_t*, uint32_t, uint32_t, uint32_t, uint8_t*, int32_t*);
    static const BulkKernel kernels[2][2] = {
        {mlf_plan_kernel_stream<MLF_PACK>, mlf_plan_kernel_bulk<MLF_PACK>},
        {mlf_plan_kernel_stream<MLF_UNPACK>, mlf_plan_kernel_bulk<MLF_UNPACK>},
    };
    // The opt-in to more than 48 KiB of dynamic shared memory is a per-device function attribute:
    // a process that drives several GPUs has to set it once on each of them.
    static std::mutex opt_mu;
    static bool opted_in[kMaxDevices] = {false};
    int dev = 0;
    MLF_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return mlf::fail(MLF_ERR_INVALID, "mlf_plan_launch: device index out of range");
    {
      std::lock_guard<std::mutex> hold(opt_mu);
      if (!opted_in[dev]) {
        for (int d = 0; d < 2; ++d)
          for (int v = 0; v < 2; ++v)
            MLF_CUDA(cudaFuncSetAttribute(kernels[d][v], cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBulkDynSmem));
        opted_in[dev] = true;
      }
    }
    const bool staged = p->nlinear < p->ntiles;
    const BulkKernel kernel = kernels[p->direction == MLF_PACK ? 0 : 1][staged ? 1 : 0];
    const int32_t rc = wave_grid(kernel, max_ctas, p->ntiles, &grid, kBulkDynSmem);
    if (rc != MLF_OK) return rc;
    if (staged) MLF_CUDA(cudaMemsetAsync(p->d_status + 1, 0, sizeof(int32_t), s));  // the staged-tile counter starts at 0
    kernel<<<grid, kThreads, kBulkDynSmem, s>>>(p->d_segs, p->d_tile_begin, p->nseg, p->nlinear, p->ntiles, image, p->d_status);
  } else {
    int32_t rc = p->direction == MLF_PACK ? wave_grid(mlf_plan_kernel<MLF_PACK>, max_ctas, p->ntiles, &grid)
                                          : wave_grid(mlf_plan_kernel<MLF_UNPACK>, max_ctas, p->ntiles, &grid);
    if (rc != MLF_OK) return rc;
    if (p->direction == MLF_PACK)
      mlf_plan_kernel<MLF_PACK><<<grid, kThreads, 0, s>>>(p->d_segs, p->d_tile_begin, p->nseg, p->ntiles, image);
    else
      mlf_plan_kernel<MLF_UNPACK><<<grid, kThreads, 0, s>>>(p->d_segs, p->d_tile_begin, p->nseg, p->ntiles, image);
  }
  MLF_CUDA(cudaGetLastError());
  mlf::g_launches.fetch_add(1);
  return MLF_OK;
}

int32_t mlf_plan_status(mlf_plan* p) {
  if (!p) return mlf::fail(MLF_ERR_INVALID, "mlf_plan_status: null plan");
  if (!p->d_status) return MLF_OK;
  int32_t v = 0;
  MLF_CUDA(cudaMemcpy(&v, p->d_status, sizeof(v), cudaMemcpyDeviceToHost));
  if (v != 0) {
    MLF_CUDA(cudaMemset(p->d_status, 0, sizeof(v)));
    return mlf::fail(v, "a plan kernel recorded status " + std::to_string(v));
  }
  return MLF_OK;
}

int32_t mlf_pack_noalloc(const mlf_copy_desc* descs, uint64_t n, void* image_base, uint64_t image_capacity, void* stream) {
  if (n > 0 && !descs) return mlf::fail(MLF_ERR_INVALID, "mlf_pack_noalloc: null descriptors");
  if (n > kNoAllocMaxSegs)
    return mlf::fail(MLF_ERR_TOO_LARGE, "mlf_pack_noalloc takes at most " + std::to_string(kNoAllocMaxSegs) +
                                            " descriptors per call, got " + std::to_string(n) +
                                            "; split the object or use mlf_plan_create");
  int dev = 0;
  MLF_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return mlf::fail(MLF_ERR_INVALID, "mlf_pack_noalloc: device index out of range");
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  std::lock_guard<std::mutex> hold(g_noalloc_mu);
  if (!g_noalloc_dev_ptr[dev]) {
    // one-time set-up for this device: ask the runtime where the static array lives here
    uint8_t* where = nullptr;
    MLF_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&where), g_noalloc_scratch));
    g_noalloc_dev_ptr[dev] = where;
  }
  uint8_t* scratch = g_noalloc_dev_ptr[dev];

  uint32_t nseg = 0;
  uint64_t tiles = 0, extent = 0;
  for (uint64_t i = 0; i < n; ++i) {
    uint64_t ntile = 0, seg_payload = 0, seg_extent = 0;
    const int32_t rc = plan_segment(descs[i], i, MLF_PACK, 0, &g_noalloc_host_segs[nseg], &ntile, &seg_payload, &seg_extent);
    if (rc != MLF_OK) return rc;
    if (ntile == 0) continue;
    extent = std::max(extent, seg_extent);
    if (tiles + ntile > 0xfffffff0ull) return mlf::fail(MLF_ERR_TOO_LARGE, "mlf_pack_noalloc: too many tiles");
    g_noalloc_host_tiles[nseg] = (uint32_t)tiles;
    tiles += ntile;
    ++nseg;
  }
  g_noalloc_host_tiles[nseg] = (uint32_t)tiles;
  if (extent > image_capacity)
    return mlf::fail(MLF_ERR_BOUNDS, "descriptors touch " + std::to_string(extent) + " image bytes but only " +
                                         std::to_string(image_capacity) + " are available");
  if (tiles == 0) return MLF_OK;
  if (!image_base) return mlf::fail(MLF_ERR_INVALID, "mlf_pack_noalloc: null image");

  // The array still holds the previous call's tables. Everything the kernel reads, entries
  // [0, nseg) and [0, nseg], is overwritten here; the status word is the one thing that must
  // start at zero. The uploads are ordered on `stream`, ahead of the kernel, and have left the
  // host staging arrays by the time cudaMemcpyAsync returns (pageable source).
  Seg* d_segs = reinterpret_cast<Seg*>(scratch);
  uint32_t* d_tiles = reinterpret_cast<uint32_t*>(scratch + kNoAllocSegBytes);
  MLF_CUDA(cudaMemsetAsync(scratch + kNoAllocStatusOff, 0, 256, s));
  MLF_CUDA(cudaMemcpyAsync(d_segs, g_noalloc_host_segs, sizeof(Seg) * nseg, cudaMemcpyHostToDevice, s));
  MLF_CUDA(cudaMemcpyAsync(d_tiles, g_noalloc_host_tiles, sizeof(uint32_t) * (nseg + 1), cudaMemcpyHostToDevice, s));
  uint32_t grid = 1;
  const int32_t rc = wave_grid(mlf_plan_kernel<MLF_PACK>, 0, tiles, &grid);
  if (rc != MLF_OK) return rc;
  mlf_plan_kernel<MLF_PACK><<<grid, kThreads, 0, s>>>(d_segs, d_tiles, nseg, (uint32_t)tiles, static_cast<uint8_t*>(image_base));
  MLF_CUDA(cudaGetLastError());
  mlf::g_launches.fetch_add(1);
  return MLF_OK;
}

int32_t mlf_selftest_wait_timeout(uint64_t budget_ns, void* stream) {
  if (budget_ns == 0 || budget_ns > 100000000ull)
    return mlf::fail(MLF_ERR_INVALID, "mlf_selftest_wait_timeout: budget must be between 1 ns and 100 ms");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int32_t* d_status = nullptr;
  MLF_CUDA(cudaMalloc(&d_status, sizeof(int32_t)));
  cudaError_t e = cudaMemsetAsync(d_status, 0, sizeof(int32_t), s);
  int32_t recorded = 0;
  if (e == cudaSuccess) {
    mlf_wait_selftest_kernel<<<1, 32, 0, s>>>(budget_ns, d_status);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaMemcpyAsync(&recorded, d_status, sizeof(int32_t), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  cudaFree(d_status);
  if (e != cudaSuccess) return mlf::cuda_fail(e, "mlf_selftest_wait_timeout");
  mlf::g_launches.fetch_add(1);
  if (recorded == MLF_ERR_TIMEOUT) return mlf::fail(MLF_ERR_TIMEOUT, "bounded device-side wait gave up after its budget (as this self-test expects)");
  return MLF_OK;
}

int32_t mlf_copy_kernel_launch(void* dst, const void* src, uint64_t nbytes, void* stream, int32_t max_ctas) {
  if (nbytes == 0) return MLF_OK;
  if (!dst || !src) return mlf::fail(MLF_ERR_INVALID, "mlf_copy_kernel_launch: null pointer");
  uint32_t grid = 1;
  int32_t rc = wave_grid(mlf_flat_copy_kernel, max_ctas, (nbytes + 127 + kTileBytes - 1) / kTileBytes, &grid);
  if (rc != MLF_OK) return rc;
  mlf_flat_copy_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src), nbytes);
  MLF_CUDA(cudaGetLastError());
  mlf::g_launches.fetch_add(1);
  return MLF_OK;
}

}  // extern "C"
