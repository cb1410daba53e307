// TRANSPOSE tiles of a copy plan: the tensor's unit-stride dimension is not the image's. Device code
// of every form (element-wise, vector, matrix, pipelined narrow rows) and the tile geometry the
// planner shares with them. Every tile function must run with kThreads threads.
#ifndef MLF_TRANSPOSE_TILES_CUH_
#define MLF_TRANSPOSE_TILES_CUH_

#include "bulk_pipeline.cuh"
#include "copy_device.cuh"
#include "plan_seg.cuh"

namespace mlf {
namespace plan {

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

}  // namespace plan
}  // namespace mlf
#endif  // MLF_TRANSPOSE_TILES_CUH_
