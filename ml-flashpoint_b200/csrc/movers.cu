// Thin entry points around CUDA runtime services: copy-engine transfers, library-owned memory,
// IPC handles for peer replication, streams and events. Kept free of any policy so that the
// Python host code decides what overlaps with what.
#include <stdlib.h>
#include <string.h>
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

// Bytes of a slot actually used per chunk. MLF_BOUNCE_CHUNK_KIB overrides the default (tuning aid):
// small chunks keep a slot inside the CPU's last-level cache between the CPU copy and the DMA read.
uint64_t chunk_bytes() {
  static const uint64_t value = []() -> uint64_t {
    const char* v = getenv("MLF_BOUNCE_CHUNK_KIB");
    uint64_t kib = v ? strtoull(v, nullptr, 10) : 0;
    if (kib == 0) kib = MLF_BOUNCE_DEFAULT_CHUNK_KIB;
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
int32_t bounce_transfer(void* dev_ptr, void* host_ptr, int fd, uint64_t file_off, uint64_t nbytes, int32_t to_device,
                        int32_t nthreads) {
  if (nbytes == 0) return MLF_OK;
  if (!dev_ptr || (!host_ptr && fd < 0)) return mlf::fail(MLF_ERR_INVALID, "bounce transfer: null pointer");
  int workers = nthreads > 0 ? nthreads : (int)std::max(1u, std::thread::hardware_concurrency() / 2);
  workers = std::min(workers, kMaxWorkers);
  const uint64_t chunk = chunk_bytes();
  const uint64_t nchunks = (nbytes + chunk - 1) / chunk;
  workers = (int)std::min<uint64_t>((uint64_t)workers, nchunks);
  int dev = 0;
  MLF_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> hold(g_ring.mu);
  MLF_CUDA(ensure_slots(workers));

  std::atomic<int> first_error{(int)cudaSuccess};
  std::atomic<bool> io_failed{false};
  auto run = [&](int w) {
    cudaError_t e = cudaSetDevice(dev);
    cudaStream_t stream = nullptr;
    cudaEvent_t done[2] = {nullptr, nullptr};
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
    for (int k = 0; k < 2 && e == cudaSuccess; ++k) e = cudaEventCreateWithFlags(&done[k], cudaEventDisableTiming);
    bool used[2] = {false, false};
    uint64_t pending_off[2] = {0, 0}, pending_len[2] = {0, 0};
    int turn = 0;
    for (uint64_t c = (uint64_t)w; c < nchunks && e == cudaSuccess; c += (uint64_t)workers, turn ^= 1) {
      const uint64_t off = c * chunk;
      const uint64_t len = std::min(chunk, nbytes - off);
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
            const ssize_t n = pread(fd, slot + got, len - got, (off_t)(file_off + off + got));
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
    if (e != cudaSuccess) {
      int expected = (int)cudaSuccess;
      first_error.compare_exchange_strong(expected, (int)e);
    }
  };
  std::vector<std::thread> pool;
  for (int w = 1; w < workers; ++w) pool.emplace_back(run, w);
  run(0);
  for (auto& t : pool) t.join();
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
  return mlf::bounce_transfer(dev_ptr, host_ptr, -1, 0, nbytes, to_device, nthreads);
}

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
