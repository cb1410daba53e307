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
#include "plan_seg.cuh"
#include "transpose_tiles.cuh"

namespace {

using namespace mlf::plan;

// ------------------------------------------------------------------------------------ device

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

// Form of the transposes in pack plans of the bulk kernels: MLF_TRANSPOSE_FORM = matrix (default) | vector | element.
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
