// File-backed, CUDA-registrable buffer object behind the mlf_buf_* entry points.
//
// Behaviour follows the reference's BufferObject (checkpoint_object_manager/buffer_object/
// buffer_object.cpp:25-198 with the file handling of buffer_helper.cpp:43-314): create with
// O_EXCL or O_TRUNC + ftruncate + mmap(MAP_SHARED), read-only open sized by fstat, resize as
// munmap/ftruncate/mmap, close with optional truncation. What is new is the page-locking
// lifecycle: a mapping can be registered with CUDA so that the pack kernel and the copy engines
// address it directly. The mapping is page-locked in chunks of kRegChunk bytes, so that resizing a
// registered buffer (a pool buffer shrunk to the object's exact size) only touches the chunks
// behind the new end instead of page-locking the whole file again; pages are never left pinned
// behind the end of a truncated file (they would be orphaned).
#include <errno.h>
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <functional>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "common.h"

#ifndef MADV_POPULATE_READ
#define MADV_POPULATE_READ 22
#endif
#ifndef MADV_POPULATE_WRITE
#define MADV_POPULATE_WRITE 23
#endif

struct mlf_buf {
  std::string id;
  void* ptr = nullptr;
  uint64_t capacity = 0;
  int fd = -1;
  bool readonly = false;
  bool closed = true;
  bool registered = false;
  uint64_t reg_chunk = 0;             // chunk size of this registration (the capacity if it is one range)
  std::vector<uint64_t> reg_lens;     // bytes page-locked in chunk i, which starts at ptr + i * reg_chunk
};

namespace {

thread_local std::string t_error = "";

int make_parent_dirs(const std::string& path) {
  size_t slash = path.find_last_of('/');
  if (slash == std::string::npos || slash == 0) return 0;
  std::string dir = path.substr(0, slash);
  for (size_t i = 1; i <= dir.size(); ++i) {
    if (i == dir.size() || dir[i] == '/') {
      std::string part = dir.substr(0, i);
      if (mkdir(part.c_str(), 0777) != 0 && errno != EEXIST) return -1;
    }
  }
  return 0;
}

// Faults every page of [p, p+n) in, several threads wide, so that page-locking afterwards does
// not take the faults one at a time.
void populate(void* p, uint64_t n, bool writable) {
  const uint64_t kMinPerThread = 256ull << 20;
  unsigned hw = std::thread::hardware_concurrency();
  uint64_t want = n / kMinPerThread;
  unsigned nthreads = (unsigned)std::max<uint64_t>(1, std::min<uint64_t>(want, std::min(hw ? hw : 1u, 16u)));
  const long page = sysconf(_SC_PAGESIZE);
  auto work = [=](uint64_t begin, uint64_t end) {
    char* base = static_cast<char*>(p) + begin;
    uint64_t len = end - begin;
    if (madvise(base, len, writable ? MADV_POPULATE_WRITE : MADV_POPULATE_READ) == 0) return;
    // Older kernels: touch one byte per page (a read is enough to instantiate a tmpfs page).
    volatile char sink = 0;
    for (uint64_t off = 0; off < len; off += page) sink += base[off];
    (void)sink;
  };
  if (nthreads == 1) {
    work(0, n);
    return;
  }
  std::vector<std::thread> pool;
  uint64_t per = ((n / nthreads) + page - 1) / page * page;
  for (unsigned t = 0; t < nthreads; ++t) {
    uint64_t b = std::min<uint64_t>(n, t * per), e = std::min<uint64_t>(n, (t + 1) * per);
    if (t == nthreads - 1) e = n;
    if (b < e) pool.emplace_back(work, b, e);
  }
  for (auto& th : pool) th.join();
}

constexpr uint64_t kRegChunk = 512ull << 20;
constexpr int32_t kNotInPlace = 1;  // internal: the mapping cannot be resized where it is

// Address ranges page-locked by this library, for cutting copies at their boundaries.
std::mutex g_locked_mu;
std::map<uintptr_t, uintptr_t> g_locked;  // start -> end

int32_t lock_range(char* p, uint64_t len, bool readonly) {
  unsigned flags = cudaHostRegisterPortable | cudaHostRegisterMapped;
  if (readonly) flags |= cudaHostRegisterReadOnly;
  cudaError_t e = cudaHostRegister(p, len, flags);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return mlf::cuda_fail(e, "cudaHostRegister");
  }
  std::lock_guard<std::mutex> hold(g_locked_mu);
  g_locked[(uintptr_t)p] = (uintptr_t)p + len;
  return MLF_OK;
}

int32_t unlock_range(char* p) {
  {
    std::lock_guard<std::mutex> hold(g_locked_mu);
    g_locked.erase((uintptr_t)p);
  }
  cudaError_t e = cudaHostUnregister(p);
  if (e != cudaSuccess) return mlf::cuda_fail(e, "cudaHostUnregister");
  return MLF_OK;
}

// Unlocks chunks from the back until `keep` chunks remain.
int32_t unlock_chunks_from(mlf_buf* b, size_t keep) {
  int32_t rc = MLF_OK;
  while (b->reg_lens.size() > keep) {
    const size_t i = b->reg_lens.size() - 1;
    const int32_t r = unlock_range(static_cast<char*>(b->ptr) + i * b->reg_chunk);
    if (r != MLF_OK && rc == MLF_OK) rc = r;
    b->reg_lens.pop_back();
  }
  return rc;
}

// Page-locks [from, capacity) of the mapping, chunk by chunk; `from` is a chunk boundary.
int32_t lock_chunks_to_end(mlf_buf* b, uint64_t from) {
  for (uint64_t at = from; at < b->capacity; at += b->reg_chunk) {
    const uint64_t len = std::min<uint64_t>(b->reg_chunk, b->capacity - at);
    const int32_t rc = lock_range(static_cast<char*>(b->ptr) + at, len, b->readonly);
    if (rc != MLF_OK) return rc;
    b->reg_lens.push_back(len);
  }
  return MLF_OK;
}

int32_t drop_registration(mlf_buf* b) {
  if (!b->registered) return MLF_OK;
  const int32_t rc = unlock_chunks_from(b, 0);
  b->registered = false;
  return rc;
}

int32_t do_register(mlf_buf* b) {
  populate(b->ptr, b->capacity, !b->readonly);
  // Kernels address the whole mapping through one device pointer. Chunks keep that property only
  // where registered host memory is addressed by its host pointer; elsewhere lock one range.
  int dev = 0, same_pointer = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&same_pointer, cudaDevAttrCanUseHostPointerForRegisteredMem, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    same_pointer = 0;
  }
  b->reg_chunk = same_pointer ? kRegChunk : std::max<uint64_t>(b->capacity, 1);
  b->reg_lens.clear();
  const int32_t rc = lock_chunks_to_end(b, 0);
  if (rc != MLF_OK) {
    (void)unlock_chunks_from(b, 0);
    return rc;
  }
  b->registered = true;
  return MLF_OK;
}

// Resizes a registered mapping without moving it: only the chunks behind the smaller of the two
// ends are unlocked and locked again. Returns kNotInPlace (nothing changed) if the mapping
// cannot grow where it is; the caller then takes the general path.
int32_t resize_registered_in_place(mlf_buf* b, uint64_t new_capacity) {
  const uint64_t chunk = b->reg_chunk;
  if (chunk != kRegChunk) return kNotInPlace;  // one-range registration
  const uint64_t old_capacity = b->capacity;
  const uint64_t edge = std::min(old_capacity, new_capacity);
  const size_t keep = (size_t)(edge / chunk);  // chunks entirely in front of the edge stay locked
  if (new_capacity > old_capacity) {
    if (ftruncate(b->fd, (off_t)new_capacity) != 0) return mlf::fail_errno(MLF_ERR_IO, "ftruncate() failed during resize of " + b->id);
    // the partial chunk at the old end is unlocked first: it will be locked again, longer
    int32_t rc = unlock_chunks_from(b, keep);
    if (rc != MLF_OK) return rc;
    void* p = mremap(b->ptr, old_capacity, new_capacity, 0);
    if (p == MAP_FAILED) {
      if (ftruncate(b->fd, (off_t)old_capacity) != 0) {
        // best effort: a longer file behind an unchanged mapping is harmless
      }
      rc = lock_chunks_to_end(b, keep * chunk);  // as before
      return rc != MLF_OK ? rc : kNotInPlace;
    }
    b->capacity = new_capacity;
    populate(static_cast<char*>(b->ptr) + keep * chunk, new_capacity - keep * chunk, true);
    return lock_chunks_to_end(b, keep * chunk);
  }
  int32_t rc = unlock_chunks_from(b, keep);
  if (rc != MLF_OK) return rc;
  if (mremap(b->ptr, old_capacity, new_capacity, 0) == MAP_FAILED)
    return mlf::fail_errno(MLF_ERR_IO, "mremap() failed during resize of " + b->id);
  b->capacity = new_capacity;
  if (ftruncate(b->fd, (off_t)new_capacity) != 0) return mlf::fail_errno(MLF_ERR_IO, "ftruncate() failed during resize of " + b->id);
  return lock_chunks_to_end(b, keep * chunk);
}

}  // namespace

namespace mlf {
void for_each_locked_piece(const void* p, uint64_t n, const std::function<void(const void*, uint64_t)>& fn) {
  uintptr_t at = (uintptr_t)p;
  const uintptr_t end = at + n;
  std::vector<std::pair<uintptr_t, uintptr_t>> cuts;
  {
    std::lock_guard<std::mutex> hold(g_locked_mu);
    auto it = g_locked.upper_bound(at);
    if (it != g_locked.begin()) --it;
    for (; it != g_locked.end() && it->first < end; ++it)
      if (it->second > at) cuts.emplace_back(it->first, it->second);
  }
  for (const auto& range : cuts) {
    if (range.first > at) {  // bytes in front of this range that are not page-locked by this library
      fn(reinterpret_cast<const void*>(at), std::min(range.first, end) - at);
      at = std::min(range.first, end);
    }
    if (at >= end) break;
    const uintptr_t stop = std::min(range.second, end);
    if (stop > at) {
      fn(reinterpret_cast<const void*>(at), stop - at);
      at = stop;
    }
  }
  if (at < end) fn(reinterpret_cast<const void*>(at), end - at);
}
}  // namespace mlf

namespace mlf {
std::atomic<uint64_t> g_launches{0};

int32_t fail(int32_t code, const std::string& msg) {
  t_error = msg;
  return code;
}
int32_t fail_errno(int32_t code, const std::string& msg) {
  t_error = msg + ": " + strerror(errno);
  return code;
}
void clear_error() { t_error.clear(); }
}  // namespace mlf

extern "C" {

const char* mlf_last_error(void) { return t_error.c_str(); }
const char* mlf_version(void) { return "mlf_b200 sm_100a"; }
uint64_t mlf_launch_count(void) { return mlf::g_launches.load(); }

int32_t mlf_buf_create(const char* object_id, uint64_t capacity, int32_t overwrite, mlf_buf** out) {
  if (!object_id || !out) return mlf::fail(MLF_ERR_INVALID, "mlf_buf_create: null argument");
  *out = nullptr;
  if (capacity == 0)
    return mlf::fail(MLF_ERR_INVALID, std::string("a buffer needs a capacity greater than 0: ") + object_id);
  std::string id(object_id);
  if (make_parent_dirs(id) != 0) return mlf::fail_errno(MLF_ERR_IO, "mkdir failed for parents of " + id);
  int flags = O_CREAT | O_RDWR | O_CLOEXEC | (overwrite ? O_TRUNC : O_EXCL);
  int fd = open(object_id, flags, 0666);
  if (fd < 0) {
    if (errno == EEXIST)
      return mlf::fail(MLF_ERR_EXISTS, "open() failed for file: " + id + ". File already exists and overwrite is set to false.");
    return mlf::fail_errno(MLF_ERR_IO, "open() failed for file: " + id);
  }
  if (ftruncate(fd, (off_t)capacity) != 0) {
    int32_t rc = mlf::fail_errno(MLF_ERR_IO, "ftruncate() failed for file: " + id);
    close(fd);
    return rc;
  }
  void* p = mmap(nullptr, capacity, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (p == MAP_FAILED) {
    int32_t rc = mlf::fail_errno(MLF_ERR_IO, "mmap() failed for file: " + id);
    close(fd);
    return rc;
  }
  mlf_buf* b = new mlf_buf();
  b->id = id;
  b->ptr = p;
  b->capacity = capacity;
  b->fd = fd;
  b->readonly = false;
  b->closed = false;
  *out = b;
  return MLF_OK;
}

int32_t mlf_buf_open_ro(const char* object_id, mlf_buf** out) {
  if (!object_id || !out) return mlf::fail(MLF_ERR_INVALID, "mlf_buf_open_ro: null argument");
  *out = nullptr;
  std::string id(object_id);
  int fd = open(object_id, O_RDONLY | O_CLOEXEC);
  if (fd < 0) return mlf::fail_errno(MLF_ERR_IO, "open() failed for file: " + id);
  struct stat st;
  if (fstat(fd, &st) != 0) {
    int32_t rc = mlf::fail_errno(MLF_ERR_IO, "fstat() failed for file: " + id);
    close(fd);
    return rc;
  }
  if (S_ISDIR(st.st_mode)) {
    close(fd);
    return mlf::fail(MLF_ERR_IO, "Path is a directory, not a file: " + id);
  }
  if (!S_ISREG(st.st_mode)) {
    close(fd);
    return mlf::fail(MLF_ERR_IO, "not a regular file: " + id);
  }
  if (st.st_size == 0) {
    close(fd);
    return mlf::fail(MLF_ERR_INVALID, "File cannot be empty, a zero-sized file cannot be mapped: " + id);
  }
  void* p = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_SHARED, fd, 0);
  if (p == MAP_FAILED) {
    int32_t rc = mlf::fail_errno(MLF_ERR_IO, "mmap() failed for file: " + id);
    close(fd);
    return rc;
  }
  mlf_buf* b = new mlf_buf();
  b->id = id;
  b->ptr = p;
  b->capacity = (uint64_t)st.st_size;
  b->fd = fd;
  b->readonly = true;
  b->closed = false;
  *out = b;
  return MLF_OK;
}

int32_t mlf_buf_resize(mlf_buf* b, uint64_t new_capacity) {
  if (!b) return mlf::fail(MLF_ERR_INVALID, "mlf_buf_resize: null buffer");
  if (b->closed) return mlf::fail(MLF_ERR_CLOSED, "cannot resize a closed buffer: " + b->id);
  if (b->readonly) return mlf::fail(MLF_ERR_READONLY, "cannot resize a read-only buffer: " + b->id);
  if (new_capacity == 0) return mlf::fail(MLF_ERR_INVALID, "cannot resize to 0 bytes: " + b->id);
  if (new_capacity == b->capacity) return MLF_OK;
  bool was_registered = b->registered;
  int32_t rc = MLF_OK;
  if (was_registered) {
    rc = resize_registered_in_place(b, new_capacity);
    if (rc != kNotInPlace) {
      if (rc != MLF_OK) {  // half-done: give the page locks up, the mapping itself is still consistent
        (void)drop_registration(b);
      }
      return rc;
    }
    mlf::clear_error();
  }
  rc = drop_registration(b);
  if (rc != MLF_OK) return rc;
  if (munmap(b->ptr, b->capacity) != 0) return mlf::fail_errno(MLF_ERR_IO, "munmap() failed during resize of " + b->id);
  b->ptr = nullptr;
  if (ftruncate(b->fd, (off_t)new_capacity) != 0) {
    rc = mlf::fail_errno(MLF_ERR_IO, "ftruncate() failed during resize of " + b->id);
    close(b->fd);
    b->fd = -1;
    b->capacity = 0;
    b->closed = true;
    return rc;
  }
  void* p = mmap(nullptr, new_capacity, PROT_READ | PROT_WRITE, MAP_SHARED, b->fd, 0);
  if (p == MAP_FAILED) {
    rc = mlf::fail_errno(MLF_ERR_IO, "mmap() failed during resize of " + b->id);
    close(b->fd);
    b->fd = -1;
    b->capacity = 0;
    b->closed = true;
    return rc;
  }
  b->ptr = p;
  b->capacity = new_capacity;
  if (was_registered) return do_register(b);
  return MLF_OK;
}

int32_t mlf_buf_close(mlf_buf* b, int64_t truncate_size) {
  if (!b) return mlf::fail(MLF_ERR_INVALID, "mlf_buf_close: null buffer");
  if (b->closed) return MLF_OK;
  int32_t rc = drop_registration(b);
  if (b->ptr && munmap(b->ptr, b->capacity) != 0 && rc == MLF_OK)
    rc = mlf::fail_errno(MLF_ERR_IO, "munmap() failed for " + b->id);
  if (truncate_size >= 0 && !b->readonly && b->fd >= 0) {
    if (ftruncate(b->fd, (off_t)truncate_size) != 0 && rc == MLF_OK)
      rc = mlf::fail_errno(MLF_ERR_IO, "ftruncate() failed while closing " + b->id);
  }
  if (b->fd >= 0 && close(b->fd) != 0 && rc == MLF_OK) rc = mlf::fail_errno(MLF_ERR_IO, "close() failed for " + b->id);
  b->ptr = nullptr;
  b->capacity = 0;
  b->fd = -1;
  b->closed = true;
  return rc;
}

void mlf_buf_destroy(mlf_buf* b) {
  if (!b) return;
  (void)mlf_buf_close(b, -1);
  delete b;
}

const char* mlf_buf_id(const mlf_buf* b) { return b ? b->id.c_str() : ""; }
uint64_t mlf_buf_capacity(const mlf_buf* b) { return (b && !b->closed) ? b->capacity : 0; }
void* mlf_buf_host_ptr(const mlf_buf* b) { return (b && !b->closed) ? b->ptr : nullptr; }
int32_t mlf_buf_is_closed(const mlf_buf* b) { return (!b || b->closed || b->fd < 0 || b->ptr == nullptr) ? 1 : 0; }
int32_t mlf_buf_is_readonly(const mlf_buf* b) { return (b && b->readonly) ? 1 : 0; }
int32_t mlf_buf_is_registered(const mlf_buf* b) { return (b && b->registered) ? 1 : 0; }

int32_t mlf_buf_register(mlf_buf* b) {
  if (!b) return mlf::fail(MLF_ERR_INVALID, "mlf_buf_register: null buffer");
  if (b->closed) return mlf::fail(MLF_ERR_CLOSED, "cannot register a closed buffer: " + b->id);
  if (b->registered) return MLF_OK;
  return do_register(b);
}

int32_t mlf_buf_unregister(mlf_buf* b) {
  if (!b) return mlf::fail(MLF_ERR_INVALID, "mlf_buf_unregister: null buffer");
  return drop_registration(b);
}

static int32_t read_to_device(const mlf_buf* b, uint64_t offset, void* dev_ptr, uint64_t nbytes, int32_t nthreads,
                              int32_t lock_run_mib) {
  if (!b) return mlf::fail(MLF_ERR_INVALID, "mlf_buf_read_to_device: null buffer");
  if (b->closed) return mlf::fail(MLF_ERR_CLOSED, "buffer is closed: " + b->id);
  if (offset > b->capacity || nbytes > b->capacity - offset)
    return mlf::fail(MLF_ERR_BOUNDS, "read of " + std::to_string(nbytes) + " bytes at " + std::to_string(offset) +
                                         " leaves the object " + b->id);
  if (b->registered) {  // page-locked already: copy-engine transfers, no CPU copy
    const char* src = static_cast<const char*>(b->ptr) + offset;
    char* dst = static_cast<char*>(dev_ptr);
    int32_t rc = MLF_OK;
    mlf::for_each_locked_piece(src, nbytes, [&](const void* piece, uint64_t len) {
      if (rc != MLF_OK) return;
      cudaError_t e = cudaMemcpyAsync(dst + (static_cast<const char*>(piece) - src), piece, len, cudaMemcpyHostToDevice, 0);
      if (e != cudaSuccess) rc = mlf::cuda_fail(e, "cudaMemcpyAsync");
    });
    if (rc != MLF_OK) return rc;
    MLF_CUDA(cudaStreamSynchronize(0));
    return MLF_OK;
  }
  // units of the bounce ring are 4 MiB unless tuned otherwise; a run is given in MiB to stay independent of that
  const uint32_t run_units = lock_run_mib > 0 ? (uint32_t)std::max<int64_t>(1, (int64_t)lock_run_mib / 4) : 0;
  return mlf::bounce_transfer(dev_ptr, nullptr, b->fd, offset, nbytes, 1, nthreads, run_units ? b->id.c_str() : nullptr, run_units);
}

int32_t mlf_buf_read_to_device(const mlf_buf* b, uint64_t offset, void* dev_ptr, uint64_t nbytes, int32_t nthreads) {
  return read_to_device(b, offset, dev_ptr, nbytes, nthreads, 0);
}

int32_t mlf_buf_read_to_device_hybrid(const mlf_buf* b, uint64_t offset, void* dev_ptr, uint64_t nbytes, int32_t nthreads,
                                      int32_t lock_run_mib) {
  if (lock_run_mib < 0) return mlf::fail(MLF_ERR_INVALID, "mlf_buf_read_to_device_hybrid: negative run size");
  return read_to_device(b, offset, dev_ptr, nbytes, nthreads, lock_run_mib);
}

int32_t mlf_buf_dev_ptr(const mlf_buf* b, void** out) {
  if (!b || !out) return mlf::fail(MLF_ERR_INVALID, "mlf_buf_dev_ptr: null argument");
  *out = nullptr;
  if (b->closed) return mlf::fail(MLF_ERR_CLOSED, "buffer is closed: " + b->id);
  if (!b->registered) return mlf::fail(MLF_ERR_INVALID, "buffer is not registered with CUDA: " + b->id);
  MLF_CUDA(cudaHostGetDevicePointer(out, b->ptr, 0));
  return MLF_OK;
}

}  // extern "C"
