// Device-side byte movers shared by the plan kernel and the flat copy kernel.
//
// Everything here is pure data movement between two byte addresses of arbitrary alignment: the
// checkpoint object format has no padding, so a tensor's payload starts at whatever byte the
// headers before it end on. The destination side is always brought to 16-byte alignment and
// written with full 16-byte vectors; a misaligned source is read as aligned 16-byte vectors and
// shifted into place in registers.
#ifndef MLF_COPY_DEVICE_CUH_
#define MLF_COPY_DEVICE_CUH_

#include <cuda_runtime.h>
#include <stdint.h>

namespace mlf {

__device__ __forceinline__ uint4 ld_vec(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// Variant that keeps the line in L1: the shifted path reads every source vector twice.
__device__ __forceinline__ uint4 ld_vec_keep(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// MLF_STORE_OP is a tuning knob of the build: the cache operator of the payload stores.
#ifndef MLF_STORE_OP
#define MLF_STORE_OP ".cs"
#endif
__device__ __forceinline__ void st_vec(uint4* p, const uint4& v) {
  asm volatile("st.global" MLF_STORE_OP ".v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// The vector held by the next higher lane (undefined for lane 31).
__device__ __forceinline__ uint4 shfl_down1(const uint4& v) {
  uint4 o;
  o.x = __shfl_down_sync(0xffffffffu, v.x, 1);
  o.y = __shfl_down_sync(0xffffffffu, v.y, 1);
  o.z = __shfl_down_sync(0xffffffffu, v.z, 1);
  o.w = __shfl_down_sync(0xffffffffu, v.w, 1);
  return o;
}

// 16 bytes starting `shift` bytes (1..15) into the 32-byte window {lo, hi}.
__device__ __forceinline__ uint4 realign(const uint4& lo, const uint4& hi, unsigned shift) {
  const unsigned bits = (shift & 3u) * 8u;
  uint4 o;
  switch (shift >> 2) {
    case 0:
      o.x = __funnelshift_r(lo.x, lo.y, bits);
      o.y = __funnelshift_r(lo.y, lo.z, bits);
      o.z = __funnelshift_r(lo.z, lo.w, bits);
      o.w = __funnelshift_r(lo.w, hi.x, bits);
      break;
    case 1:
      o.x = __funnelshift_r(lo.y, lo.z, bits);
      o.y = __funnelshift_r(lo.z, lo.w, bits);
      o.z = __funnelshift_r(lo.w, hi.x, bits);
      o.w = __funnelshift_r(hi.x, hi.y, bits);
      break;
    case 2:
      o.x = __funnelshift_r(lo.z, lo.w, bits);
      o.y = __funnelshift_r(lo.w, hi.x, bits);
      o.z = __funnelshift_r(hi.x, hi.y, bits);
      o.w = __funnelshift_r(hi.y, hi.z, bits);
      break;
    default:
      o.x = __funnelshift_r(lo.w, hi.x, bits);
      o.y = __funnelshift_r(hi.x, hi.y, bits);
      o.z = __funnelshift_r(hi.y, hi.z, bits);
      o.w = __funnelshift_r(hi.z, hi.w, bits);
      break;
  }
  return o;
}

// Copies `len` bytes from `src` to `dst` with a group of `nthr` threads (a CTA or a warp);
// `tid` is the caller's index in the group. Any alignment, any length, no overlap.
// Reads never leave the 16-byte granules that hold at least one source byte.
__device__ __forceinline__ void copy_bytes(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src, uint64_t len,
                                           unsigned tid, unsigned nthr) {
  // bring the destination to a 128-byte line for long runs (every warp store then covers whole
  // lines), to 16 bytes for short ones
  const unsigned want = len >= 1024 ? 128u : 16u;
  const unsigned head = (unsigned)min((uint64_t)((want - (unsigned)((uintptr_t)dst & (want - 1u))) & (want - 1u)), len);
  for (unsigned k = tid; k < head; k += nthr) dst[k] = src[k];
  dst += head;
  src += head;
  len -= head;
  const uint64_t nvec = len >> 4;
  const unsigned shift = (unsigned)((uintptr_t)src & 15u);
  uint4* __restrict__ d4 = reinterpret_cast<uint4*>(dst);
  if (shift == 0) {
    const uint4* __restrict__ s4 = reinterpret_cast<const uint4*>(src);
    uint64_t i = tid;
    const uint64_t step = (uint64_t)nthr * 4;
    for (; i + 3ull * nthr < nvec; i += step) {
      uint4 a = ld_vec(s4 + i);
      uint4 b = ld_vec(s4 + i + nthr);
      uint4 c = ld_vec(s4 + i + 2ull * nthr);
      uint4 d = ld_vec(s4 + i + 3ull * nthr);
      st_vec(d4 + i, a);
      st_vec(d4 + i + nthr, b);
      st_vec(d4 + i + 2ull * nthr, c);
      st_vec(d4 + i + 3ull * nthr, d);
    }
    for (; i < nvec; i += nthr) st_vec(d4 + i, ld_vec(s4 + i));
  } else {
    // Shifted source: output vector i needs aligned source vectors i and i+1. In the main loop a
    // lane takes vector i+1 from its right neighbour's registers; only lane 31 loads it.
    const uint4* __restrict__ s4 = reinterpret_cast<const uint4*>(src - shift);
    const unsigned lane = tid & 31u;
    uint64_t i = tid;
    const uint64_t step = (uint64_t)nthr * 2;
    // warp-uniform bound: all 32 lanes of the warp must be inside for the shuffles
    for (; (i - lane) + (uint64_t)nthr + 31u < nvec; i += step) {
      uint4 a = ld_vec(s4 + i);
      uint4 b = ld_vec(s4 + i + nthr);
      uint4 an = a, bn = b;
      if (lane == 31u) {
        an = ld_vec(s4 + i + 1);
        bn = ld_vec(s4 + i + nthr + 1);
      }
      const uint4 as = shfl_down1(a), bs = shfl_down1(b);
      if (lane != 31u) {
        an = as;
        bn = bs;
      }
      st_vec(d4 + i, realign(a, an, shift));
      st_vec(d4 + i + nthr, realign(b, bn, shift));
    }
    for (; i < nvec; i += nthr) {
      uint4 a0 = ld_vec_keep(s4 + i), a1 = ld_vec_keep(s4 + i + 1);
      st_vec(d4 + i, realign(a0, a1, shift));
    }
  }
  const unsigned tail = (unsigned)(len & 15u);
  if (tid < tail) {
    const uint64_t o = (nvec << 4) + tid;
    dst[o] = src[o];
  }  // tail < 16 <= nthr
}

}  // namespace mlf
#endif  // MLF_COPY_DEVICE_CUH_
