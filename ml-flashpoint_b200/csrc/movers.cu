// Thin entry points around CUDA runtime services: copy-engine transfers, library-owned memory,
// IPC handles for peer replication, streams and events. Kept free of any policy so that the
// Python host code decides what overlaps with what.
#include <string.h>

#include <string>

#include "common.h"

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
  MLF_CUDA(cudaMemcpyAsync(dst, src, nbytes, k, static_cast<cudaStream_t>(stream)));
  return MLF_OK;
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
