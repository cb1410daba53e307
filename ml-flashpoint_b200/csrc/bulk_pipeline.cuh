// Shared-memory staging ring fed by bulk asynchronous copies (cp.async.bulk + mbarrier).
//
// One elected thread streams the source of linear tiles into a ring of shared-memory slots with
// the bulk-copy engine; every thread of the CTA then reads the slot, shifts the bytes into
// destination alignment and stores 16-byte vectors. The bytes in flight live in shared memory,
// not in registers, so a CTA keeps kStages x 16 KiB of loads outstanding with a handful of
// registers per thread.
//
// Every wait is bounded: a wait that does not complete within kWaitBudgetNs records
// MLF_ERR_TIMEOUT in the caller's status word and makes the CTA leave its loop, after a second
// bounded wait for the copies it still has in flight.
#ifndef MLF_BULK_PIPELINE_CUH_
#define MLF_BULK_PIPELINE_CUH_

#include <cuda_runtime.h>
#include <stdint.h>

#include "copy_device.cuh"

namespace mlf {

#ifndef MLF_RING_STAGES
#define MLF_RING_STAGES 4
#endif
#ifndef MLF_RING_STAGE_KIB
#define MLF_RING_STAGE_KIB 16
#endif
constexpr uint32_t kStages = MLF_RING_STAGES;
constexpr uint32_t kStageBytes = MLF_RING_STAGE_KIB * 1024;
constexpr uint32_t kSlotBytes = kStageBytes + 16;  // one extra granule for a shifted source
constexpr uint64_t kWaitBudgetNs = 2000000000ull;  // 2 s: five orders of magnitude above a slot fill

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Waits for the phase with the given parity. Returns false if the time budget ran out.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint64_t budget_ns = kWaitBudgetNs) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t start = global_ns();
  for (;;) {
#pragma unroll 1
    for (int spin = 0; spin < 64; ++spin)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_ns() - start > budget_ns) return false;
  }
}
// Global -> shared bulk copy of `bytes` (multiple of 16; both addresses 16-byte aligned),
// completion counted on `bar`.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
#ifdef MLF_BULK_L2_EVICT_FIRST
  // tuning variant: the source lines are read once, so they may leave L2 first
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(smem_addr(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar)), "l"(policy)
      : "memory");
#else
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
      : "memory");
#endif
}

__device__ __forceinline__ uint4 lds_vec(const uint8_t* slot, uint32_t vec_index) {
  return *reinterpret_cast<const uint4*>(slot + (size_t)vec_index * 16);
}

// Moves one filled slot to global memory. The slot holds the aligned source granules of the
// stage: slot[shift + k] is source byte k, k in [0, len). `dst` is the destination of byte 0.
__device__ __forceinline__ void drain_slot(uint8_t* __restrict__ dst, const uint8_t* __restrict__ slot, uint32_t shift,
                                           uint32_t len, unsigned tid, unsigned nthr) {
  const uint32_t head = min((16u - (uint32_t)((uintptr_t)dst & 15u)) & 15u, len);
  if (tid < head) dst[tid] = slot[shift + tid];
  const uint32_t q = shift + head;  // slot offset of the first vectorised byte
  const uint32_t v0 = q >> 4, sh = q & 15u;
  const uint32_t nvec = (len - head) >> 4;
  uint4* __restrict__ d4 = reinterpret_cast<uint4*>(dst + head);
  if (sh == 0) {
#pragma unroll 4
    for (uint32_t i = tid; i < nvec; i += nthr) st_vec(d4 + i, lds_vec(slot, v0 + i));
  } else {
#pragma unroll 4
    for (uint32_t i = tid; i < nvec; i += nthr) st_vec(d4 + i, realign(lds_vec(slot, v0 + i), lds_vec(slot, v0 + i + 1), sh));
  }
  const uint32_t tail = (len - head) & 15u;
  if (tid < tail) {
    const uint32_t o = head + (nvec << 4) + tid;
    dst[o] = slot[shift + o];
  }
}

}  // namespace mlf
#endif  // MLF_BULK_PIPELINE_CUH_
