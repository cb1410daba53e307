// Thin entry points around CUDA runtime services: copy-engine transfers, library-owned memory,
// IPC handles for peer replication, streams and events. Kept free of any policy so that the
// Python host code decides what overlaps with what.
#include <fcntl.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "common.h"

#ifndef MLF_BOUNCE_DEFAULT_CHUNK_KIB
#define MLF_BOUNCE_DEFAULT_CHUNK_KIB 4096  // measured best on a 16-core host: 51 GB/s vs 37 GB/s at 16 MiB
#endif

namespace {

// Page-locked bounce slots for transfers to or from host memory that is NOT registered with CUDA
// (a read-only object mapping opened after a restart cannot be registered, and registering costs
// more than the transfer for anything read once). Each worker thread owns two slots and
// alternates: the CPU fills/drains one while the copy engine works on the other.
constexpr uint64_t kSlotBytes = 16ull << 20;  // upper bound of a slot
constexpr int kMaxWorkers = 32;

// Bytes of a slot actually used per chunk. Small chunks keep a slot inside the CPU's last-level cache
// between the CPU copy and the DMA read; very small ones pay per-transfer driver overhead. Measured
// on B200 hosts (restore feed, all ranks of the host at once): one rank with 16 threads 50 / 48 / 43 /
// 29 GB/s for 4 / 2 / 1 / 0.5 MiB chunks; four ranks with 8 threads each 64 / 81 / 66 GB/s in total for
// 4 / 1 / 0.25 MiB. Hence the default: 4 MiB divided by the ranks that share the host (LOCAL_WORLD_SIZE),
// not below 1 MiB. MLF_BOUNCE_CHUNK_KIB overrides it (tuning aid).
uint64_t chunk_bytes() {
  static const uint64_t value = []() -> uint64_t {
    const char* v = getenv("MLF_BOUNCE_CHUNK_KIB");
    uint64_t kib = v ? strtoull(v, nullptr, 10) : 0;
    if (kib == 0) {
      const char* w = getenv("LOCAL_WORLD_SIZE");
      const uint64_t ranks = std::max<uint64_t>(1, w ? strtoull(w, nullptr, 10) : 1);
      kib = std::max<uint64_t>(1024, MLF_BOUNCE_DEFAULT_CHUNK_KIB / ranks);
    }
    return std::min<uint64_t>(kSlotBytes, std::max<uint64_t>(64, kib) << 10);
  }();
  return value;
}

struct BounceRing {
  std::mutex mu;          // one pipelined copy at a time per process
  void* slots[kMaxWorkers * 2] = {nullptr};
  int device = -1;
};
BounceRing g_ring;
std::atomic<uint64_t> g_last_lane_bytes{0};  // bytes the lock lane moved in the most recent transfer

cudaError_t ensure_slots(int workers) {
  for (int i = 0; i < workers * 2; ++i) {
    if (g_ring.slots[i]) continue;
    cudaError_t e = cudaHostAlloc(&g_ring.slots[i], chunk_bytes(), cudaHostAllocPortable);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

}  // namespace

extern "C" {

int32_t mlf_memcpy_async(void* dst, const void* src, uint64_t nbytes, int32_t kind, void* stream) {
  if (nbytes == 0) return MLF_OK;
  if (!dst || !src) return mlf::fail(MLF_ERR_INVALID, "mlf_memcpy_async: null pointer");
  cudaMemcpyKind k;
  switch (kind) {
    case MLF_COPY_D2H: k = cudaMemcpyDeviceToHost; break;
    case MLF_COPY_H2D: k = cudaMemcpyHostToDevice; break;
    case MLF_COPY_D2D: k = cudaMemcpyDeviceToDevice; break;
    default: return mlf::fail(MLF_ERR_INVALID, "mlf_memcpy_async: unknown copy kind");
  }
  if (k == cudaMemcpyDeviceToDevice) {
    MLF_CUDA(cudaMemcpyAsync(dst, src, nbytes, k, static_cast<cudaStream_t>(stream)));
    return MLF_OK;
  }
  // a page-locked mapping is locked in chunks: one transfer per chunk it touches
  const char* host = static_cast<const char*>(k == cudaMemcpyDeviceToHost ? dst : src);
  int32_t rc = MLF_OK;
  mlf::for_each_locked_piece(host, nbytes, [&](const void* piece, uint64_t len) {
    if (rc != MLF_OK) return;
    const uint64_t off = (uint64_t)(static_cast<const char*>(piece) - host);
    cudaError_t e = cudaMemcpyAsync(static_cast<char*>(dst) + off, static_cast<const char*>(src) + off, len, k,
                                    static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) rc = mlf::cuda_fail(e, "cudaMemcpyAsync");
  });
  return rc;
}

}  // extern "C"

namespace mlf {
// Shared body of mlf_bounce_copy and mlf_buf_read_to_device. The host side is either a mapped
// address (`host_ptr`) or, for host -> device only, a file descriptor read with pread() at
// `file_off`: reading through the descriptor copies straight from the page cache into the
// page-locked slot and never builds (or tears down) page tables for the object.
//
// The range is cut into units on a grid of chunk_bytes() in the source's own address space (file
// offsets for a descriptor), so that unit boundaries fall on page boundaries of the file. Units are
// handed out dynamically from one shared range: the bounce workers take single units from the
// front; an optional "lock lane" (`lock_path` given, host -> device only) takes runs of units from
// the back, page-locks that piece of a writable mapping of the file, lets a copy engine read it in
// place and unlocks it again, one piece ahead of the transfer of the previous one. The two kinds of
// worker meet wherever their speeds put the meeting point. Page-locking costs a core far less per
// byte than pread() does, but the driver serialises it within a process, hence one lane.
int32_t bounce_transfer(void* dev_ptr, void* host_ptr, int fd, uint64_t file_off, uint64_t nbytes, int32_t to_device,
                        int32_t nthreads, const char* lock_path, uint32_t lock_run_units) {
  if (nbytes == 0) return MLF_OK;
  if (!dev_ptr || (!host_ptr && fd < 0)) return mlf::fail(MLF_ERR_INVALID, "bounce transfer: null pointer");
  // nthreads < 0 (with a lock lane): the pread threads stand back and only move what the lane leaves
  // behind when it cannot run; the lane then works alone, from the back of the range to its front
  const bool lane_only = nthreads < 0 && lock_path && lock_run_units > 0;
  int workers = nthreads > 0 ? nthreads : (int)std::max(1u, std::thread::hardware_concurrency() / 2);
  workers = std::min(workers, kMaxWorkers);
  const uint64_t chunk = chunk_bytes();
  const uint64_t space0 = fd >= 0 ? file_off : 0;  // first byte in the source's address space
  const uint64_t space1 = space0 + nbytes;
  const uint64_t unit0 = space0 / chunk, unit1 = (space1 + chunk - 1) / chunk;
  workers = (int)std::min<uint64_t>((uint64_t)workers, unit1 - unit0);
  const bool lane_wanted = lock_path && to_device && fd >= 0 && lock_run_units > 0 &&
                           (lane_only || (unit1 - unit0) >= 4ull * lock_run_units);
  int dev = 0;
  MLF_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> hold(g_ring.mu);
  MLF_CUDA(ensure_slots(workers));

  std::mutex claim_mu;
  uint64_t next_front = unit0, next_back = unit1;  // unclaimed units: [next_front, next_back)
  auto claim_front = [&](uint64_t* u) {
    std::lock_guard<std::mutex> g(claim_mu);
    if (next_front >= next_back) return false;
    *u = next_front++;
    return true;
  };
  auto claim_back = [&](uint64_t* lo, uint64_t* hi) {
    std::lock_guard<std::mutex> g(claim_mu);
    if (next_front >= next_back) return false;
    *hi = next_back;
    *lo = next_back - std::min<uint64_t>(lock_run_units, next_back - next_front);
    next_back = *lo;
    return true;
  };
  auto unit_range = [&](uint64_t lo_unit, uint64_t hi_unit, uint64_t* begin, uint64_t* len) {
    const uint64_t b = std::max(space0, lo_unit * chunk), e = std::min(space1, hi_unit * chunk);
    *begin = b;
    *len = e - b;
  };

  std::atomic<int> first_error{(int)cudaSuccess};
  std::atomic<bool> io_failed{false};
  std::atomic<uint64_t> lane_bytes{0};
  auto note_error = [&](cudaError_t e) {
    if (e == cudaSuccess) return;
    int expected = (int)cudaSuccess;
    first_error.compare_exchange_strong(expected, (int)e);
  };
  auto run = [&](int w) {
    cudaError_t e = cudaSetDevice(dev);
    cudaStream_t stream = nullptr;
    cudaEvent_t done[2] = {nullptr, nullptr};
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
    for (int k = 0; k < 2 && e == cudaSuccess; ++k) e = cudaEventCreateWithFlags(&done[k], cudaEventDisableTiming);
    bool used[2] = {false, false};
    uint64_t pending_off[2] = {0, 0}, pending_len[2] = {0, 0};
    int turn = 0;
    uint64_t u = 0;
    for (; e == cudaSuccess && claim_front(&u); turn ^= 1) {
      uint64_t begin = 0, len = 0;
      unit_range(u, u + 1, &begin, &len);
      const uint64_t off = begin - space0;  // offset in the device range (and in host_ptr)
      char* slot = static_cast<char*>(g_ring.slots[w * 2 + turn]);
      if (used[turn]) {
        e = cudaEventSynchronize(done[turn]);  // the slot's previous transfer has left (or arrived)
        if (e != cudaSuccess) break;
        if (!to_device) memcpy(static_cast<char*>(host_ptr) + pending_off[turn], slot, pending_len[turn]);
      }
      if (to_device) {
        if (fd >= 0) {
          uint64_t got = 0;
          while (got < len) {
            const ssize_t n = pread(fd, slot + got, len - got, (off_t)(begin + got));
            if (n <= 0) {
              io_failed.store(true);
              break;
            }
            got += (uint64_t)n;
          }
          if (io_failed.load()) break;
        } else {
          memcpy(slot, static_cast<const char*>(host_ptr) + off, len);
        }
        e = cudaMemcpyAsync(static_cast<char*>(dev_ptr) + off, slot, len, cudaMemcpyHostToDevice, stream);
      } else {
        e = cudaMemcpyAsync(slot, static_cast<const char*>(dev_ptr) + off, len, cudaMemcpyDeviceToHost, stream);
        pending_off[turn] = off;
        pending_len[turn] = len;
      }
      if (e == cudaSuccess) e = cudaEventRecord(done[turn], stream);
      used[turn] = true;
    }
    if (e == cudaSuccess && stream) e = cudaStreamSynchronize(stream);
    if (e == cudaSuccess && !to_device) {
      // drain what is still parked in the slots, oldest first
      for (int k = 0; k < 2; ++k) {
        const int t = turn ^ k;
        if (used[t] && pending_len[t]) {
          memcpy(static_cast<char*>(host_ptr) + pending_off[t], g_ring.slots[w * 2 + t], pending_len[t]);
          pending_len[t] = 0;
        }
      }
    }
    for (int k = 0; k < 2; ++k)
      if (done[k]) cudaEventDestroy(done[k]);
    if (stream) cudaStreamDestroy(stream);
    note_error(e);
  };

  // The lock lane. Any failure to set it up (the file cannot be opened for writing, the mapping
  // cannot be locked) simply ends the lane: the bounce workers take the rest of the range.
  auto lane = [&]() {
    if (cudaSetDevice(dev) != cudaSuccess) return;
    const int wfd = open(lock_path, O_RDWR | O_CLOEXEC);
    if (wfd < 0) return;
    const uint64_t page = (uint64_t)sysconf(_SC_PAGESIZE);
    const uint64_t map_len = (space1 + page - 1) / page * page;
    void* map = mmap(nullptr, map_len, PROT_READ | PROT_WRITE, MAP_SHARED, wfd, 0);
    close(wfd);
    if (map == MAP_FAILED) return;
    cudaStream_t stream = nullptr;
    cudaEvent_t done[2] = {nullptr, nullptr};
    cudaError_t e = cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
    for (int k = 0; k < 2 && e == cudaSuccess; ++k) e = cudaEventCreateWithFlags(&done[k], cudaEventDisableTiming);
    char* locked[2] = {nullptr, nullptr};
    int turn = 0;
    bool give_up = false;
    uint64_t lo = 0, hi = 0;
    while (e == cudaSuccess && !give_up && claim_back(&lo, &hi)) {
      uint64_t begin = 0, len = 0;
      unit_range(lo, hi, &begin, &len);
      if (locked[turn]) {  // two pieces in flight at most: finish and unlock the older one
        e = cudaEventSynchronize(done[turn]);
        if (e == cudaSuccess) e = cudaHostUnregister(locked[turn]);
        locked[turn] = nullptr;
        if (e != cudaSuccess) break;
      }
      // page-aligned outwards: inner boundaries lie on the unit grid, only the two ends of the whole
      // transfer can be ragged, and no other piece shares their pages
      const uint64_t lock_begin = begin / page * page, lock_end = std::min(map_len, (begin + len + page - 1) / page * page);
      char* piece = static_cast<char*>(map) + lock_begin;
      cudaError_t le = cudaHostRegister(piece, lock_end - lock_begin, cudaHostRegisterPortable);
      if (le != cudaSuccess) {
        // cannot lock (limits, or memory that cannot be pinned): move this piece the plain way and stop
        (void)cudaGetLastError();
        e = cudaMemcpyAsync(static_cast<char*>(dev_ptr) + (begin - space0), static_cast<char*>(map) + begin, len,
                            cudaMemcpyHostToDevice, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        give_up = true;
        break;
      }
      locked[turn] = piece;
      e = cudaMemcpyAsync(static_cast<char*>(dev_ptr) + (begin - space0), static_cast<char*>(map) + begin, len,
                          cudaMemcpyHostToDevice, stream);
      if (e == cudaSuccess) e = cudaEventRecord(done[turn], stream);
      lane_bytes.fetch_add(len);
      turn ^= 1;
    }
    if (stream) {
      cudaError_t se = cudaStreamSynchronize(stream);
      if (e == cudaSuccess) e = se;
    }
    for (int k = 0; k < 2; ++k) {
      if (locked[k]) {
        cudaError_t ue = cudaHostUnregister(locked[k]);
        if (e == cudaSuccess) e = ue;
      }
      if (done[k]) cudaEventDestroy(done[k]);
    }
    if (stream) cudaStreamDestroy(stream);
    munmap(map, map_len);
    note_error(e);
  };

  std::vector<std::thread> pool;
  if (lane_wanted && lane_only) {
    lane();  // alone; whatever it could not take (no write access, locking refused) is left for the threads
  } else if (lane_wanted) {
    pool.emplace_back(lane);
  }
  for (int w = 1; w < workers; ++w) pool.emplace_back(run, w);
  run(0);
  for (auto& t : pool) t.join();
  g_last_lane_bytes.store(lane_bytes.load());
  if (first_error.load() != (int)cudaSuccess) {
    (void)cudaGetLastError();
    return mlf::cuda_fail((cudaError_t)first_error.load(), "pipelined bounce copy");
  }
  if (io_failed.load()) return mlf::fail_errno(MLF_ERR_IO, "pread() failed or hit end of file during a bounce transfer");
  return MLF_OK;
}
}  // namespace mlf

extern "C" {

int32_t mlf_bounce_copy(void* dev_ptr, void* host_ptr, uint64_t nbytes, int32_t to_device, int32_t nthreads) {
  if (nbytes > 0 && !host_ptr) return mlf::fail(MLF_ERR_INVALID, "mlf_bounce_copy: null pointer");
  return mlf::bounce_transfer(dev_ptr, host_ptr, -1, 0, nbytes, to_device, nthreads, nullptr, 0);
}

uint64_t mlf_last_lock_lane_bytes(void) { return g_last_lane_bytes.load(); }

int32_t mlf_dev_alloc(uint64_t nbytes, void** out) {
  if (!out) return mlf::fail(MLF_ERR_INVALID, "mlf_dev_alloc: null out");
  *out = nullptr;
  if (nbytes == 0) return mlf::fail(MLF_ERR_INVALID, "mlf_dev_alloc: zero bytes");
  MLF_CUDA(cudaMalloc(out, nbytes));
  return MLF_OK;
}
int32_t mlf_dev_free(void* p) {
  if (!p) return MLF_OK;
  MLF_CUDA(cudaFree(p));
  return MLF_OK;
}
int32_t mlf_host_alloc(uint64_t nbytes, void** out) {
  if (!out) return mlf::fail(MLF_ERR_INVALID, "mlf_host_alloc: null out");
  *out = nullptr;
  if (nbytes == 0) return mlf::fail(MLF_ERR_INVALID, "mlf_host_alloc: zero bytes");
  MLF_CUDA(cudaHostAlloc(out, nbytes, cudaHostAllocPortable | cudaHostAllocMapped));
  return MLF_OK;
}
int32_t mlf_host_free(void* p) {
  if (!p) return MLF_OK;
  MLF_CUDA(cudaFreeHost(p));
  return MLF_OK;
}

int32_t mlf_ipc_export(void* dev_ptr, uint8_t handle_out[MLF_IPC_HANDLE_BYTES]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == MLF_IPC_HANDLE_BYTES, "IPC handle size");
  if (!dev_ptr || !handle_out) return mlf::fail(MLF_ERR_INVALID, "mlf_ipc_export: null argument");
  cudaIpcMemHandle_t h;
  MLF_CUDA(cudaIpcGetMemHandle(&h, dev_ptr));
  memcpy(handle_out, &h, sizeof(h));
  return MLF_OK;
}
int32_t mlf_ipc_open(const uint8_t handle[MLF_IPC_HANDLE_BYTES], void** out) {
  if (!handle || !out) return mlf::fail(MLF_ERR_INVALID, "mlf_ipc_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  MLF_CUDA(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
  return MLF_OK;
}
int32_t mlf_ipc_close(void* p) {
  if (!p) return MLF_OK;
  MLF_CUDA(cudaIpcCloseMemHandle(p));
  return MLF_OK;
}
int32_t mlf_enable_peer_access(int32_t peer_device) {
  int dev = 0, can = 0;
  MLF_CUDA(cudaGetDevice(&dev));
  if (dev == peer_device) return MLF_OK;
  MLF_CUDA(cudaDeviceCanAccessPeer(&can, dev, peer_device));
  if (!can) return mlf::fail(MLF_ERR_CUDA, "device " + std::to_string(dev) + " cannot access peer " + std::to_string(peer_device));
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    (void)cudaGetLastError();
    return MLF_OK;
  }
  MLF_CUDA(e);
  return MLF_OK;
}

int32_t mlf_set_device(int32_t device) {
  MLF_CUDA(cudaSetDevice(device));
  return MLF_OK;
}
int32_t mlf_get_device(int32_t* device) {
  if (!device) return mlf::fail(MLF_ERR_INVALID, "mlf_get_device: null out");
  int d = 0;
  MLF_CUDA(cudaGetDevice(&d));
  *device = d;
  return MLF_OK;
}
int32_t mlf_device_sm_count(int32_t* out) {
  if (!out) return mlf::fail(MLF_ERR_INVALID, "mlf_device_sm_count: null out");
  int dev = 0, sms = 0;
  MLF_CUDA(cudaGetDevice(&dev));
  MLF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  *out = sms;
  return MLF_OK;
}
int32_t mlf_stream_create(void** out) {
  if (!out) return mlf::fail(MLF_ERR_INVALID, "mlf_stream_create: null out");
  cudaStream_t s;
  MLF_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *out = s;
  return MLF_OK;
}
int32_t mlf_stream_destroy(void* stream) {
  if (!stream) return MLF_OK;
  MLF_CUDA(cudaStreamDestroy(static_cast<cudaStream_t>(stream)));
  return MLF_OK;
}
int32_t mlf_stream_sync(void* stream) {
  MLF_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return MLF_OK;
}
int32_t mlf_stream_wait_event(void* stream, void* event) {
  if (!event) return mlf::fail(MLF_ERR_INVALID, "mlf_stream_wait_event: null event");
  MLF_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0));
  return MLF_OK;
}
int32_t mlf_event_create(void** out) {
  if (!out) return mlf::fail(MLF_ERR_INVALID, "mlf_event_create: null out");
  cudaEvent_t e;
  MLF_CUDA(cudaEventCreate(&e));
  *out = e;
  return MLF_OK;
}
int32_t mlf_event_destroy(void* event) {
  if (!event) return MLF_OK;
  MLF_CUDA(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
  return MLF_OK;
}
int32_t mlf_event_record(void* event, void* stream) {
  if (!event) return mlf::fail(MLF_ERR_INVALID, "mlf_event_record: null event");
  MLF_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
  return MLF_OK;
}
int32_t mlf_event_sync(void* event) {
  if (!event) return mlf::fail(MLF_ERR_INVALID, "mlf_event_sync: null event");
  MLF_CUDA(cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
  return MLF_OK;
}
int32_t mlf_event_query(void* event) {
  if (!event) return mlf::fail(MLF_ERR_INVALID, "mlf_event_query: null event");
  cudaError_t e = cudaEventQuery(static_cast<cudaEvent_t>(event));
  if (e == cudaSuccess) return 1;
  if (e == cudaErrorNotReady) {
    (void)cudaGetLastError();
    return 0;
  }
  return mlf::cuda_fail(e, "cudaEventQuery");
}
int32_t mlf_event_elapsed_ms(void* start, void* stop, float* ms) {
  if (!start || !stop || !ms) return mlf::fail(MLF_ERR_INVALID, "mlf_event_elapsed_ms: null argument");
  MLF_CUDA(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)));
  return MLF_OK;
}

}  // extern "C"
