// Shared helpers for the C-ABI translation units: thread-local error text and CUDA call checks.
#ifndef MLF_COMMON_H_
#define MLF_COMMON_H_

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <functional>
#include <string>

#include "mlf_b200.h"

namespace mlf {

// Stores `msg` for mlf_last_error() on this thread and returns `code`.
int32_t fail(int32_t code, const std::string& msg);
// errno-flavoured variant: appends ": <strerror(errno)>".
int32_t fail_errno(int32_t code, const std::string& msg);
void clear_error();

extern std::atomic<uint64_t> g_launches;

int32_t bounce_transfer(void* dev_ptr, void* host_ptr, int fd, uint64_t file_off, uint64_t nbytes, int32_t to_device,
                        int32_t nthreads, const char* lock_path, uint32_t lock_run_units);

// Calls fn(piece, length) for consecutive pieces of the host range [p, p + n), cut wherever a
// range page-locked by this library starts or ends: a copy-engine transfer must stay inside one
// page-locked range to be treated as such.
void for_each_locked_piece(const void* p, uint64_t n, const std::function<void(const void*, uint64_t)>& fn);

inline int32_t cuda_fail(cudaError_t e, const char* what) {
  return fail(MLF_ERR_CUDA, std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")");
}

}  // namespace mlf

#define MLF_CUDA(call)                                       \
  do {                                                       \
    cudaError_t _e = (call);                                 \
    if (_e != cudaSuccess) return mlf::cuda_fail(_e, #call); \
  } while (0)

#endif  // MLF_COMMON_H_
