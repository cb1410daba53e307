/*
 * mlf_b200.h - C ABI of the B200 data path for ML Flashpoint checkpoint objects.
 *
 * One shared library (libmlf_b200.so) exports everything below with C linkage. Signatures use
 * plain pointers and integer sizes only; CUDA handles (streams, events) cross as `void*` so a
 * caller needs no CUDA headers. Every function that can fail returns an int32 status: 0 on
 * success, a negative MLF_ERR_* otherwise, and records a human-readable message retrievable with
 * mlf_last_error() on the same thread. No exception ever crosses this boundary.
 *
 * Each group names the interface of the reference implementation (google/ml-flashpoint, paths
 * relative to src/ml_flashpoint/) that it stands in for.
 */
#ifndef MLF_B200_H_
#define MLF_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ status codes */
#define MLF_OK 0
#define MLF_ERR_INVALID (-1)     /* bad argument */
#define MLF_ERR_IO (-2)          /* open/ftruncate/mmap/... failed; message carries errno text */
#define MLF_ERR_CUDA (-3)        /* a CUDA runtime call failed; message carries its error string */
#define MLF_ERR_BOUNDS (-4)      /* a descriptor would touch bytes outside the image window */
#define MLF_ERR_CLOSED (-5)      /* operation on a closed buffer */
#define MLF_ERR_EXISTS (-6)      /* create without overwrite found an existing file */
#define MLF_ERR_TIMEOUT (-7)     /* a bounded device-side wait ran out; the context stays usable */
#define MLF_ERR_TOO_LARGE (-8)   /* request exceeds a fixed capacity of the entry point */
#define MLF_ERR_READONLY (-9)    /* write-type operation on a read-only mapping */

/* Message for the last failure on the calling thread (never NULL). */
const char* mlf_last_error(void);
/* Library build tag, e.g. "mlf_b200 sm_100a". */
const char* mlf_version(void);

/* ------------------------------------------------------------------ buffer objects
 * Replaces the pybind11 class `BufferObject`
 * (checkpoint_object_manager/buffer_object/buffer_object.h:24-85, bindings.cpp:27-100;
 * file handling in buffer_helper.cpp:43-314): a file mapped MAP_SHARED that backs one
 * checkpoint object. Added here: the mapping can be page-locked and mapped into the CUDA
 * address space so kernels and copy engines write checkpoint bytes into it directly. */
typedef struct mlf_buf mlf_buf;

/* BufferObject(object_id, capacity, overwrite): create (O_EXCL unless overwrite, then O_TRUNC),
 * size with ftruncate and map read-write. Creates parent directories. capacity must be > 0. */
int32_t mlf_buf_create(const char* object_id, uint64_t capacity, int32_t overwrite, mlf_buf** out);
/* BufferObject(object_id): open an existing non-empty file read-only; capacity = file size. */
int32_t mlf_buf_open_ro(const char* object_id, mlf_buf** out);
/* resize(new_capacity): unmap, ftruncate, map again. The address may change. A CUDA registration
 * is dropped first and re-established afterwards if one was active. */
int32_t mlf_buf_resize(mlf_buf* b, uint64_t new_capacity);
/* close(truncate_size): unmap, optionally ftruncate (truncate_size >= 0, writable only), close the
 * descriptor. Idempotent; never fails hard (problems are reported through the status only). */
int32_t mlf_buf_close(mlf_buf* b, int64_t truncate_size);
/* Destructor: closes if needed and frees the handle. */
void mlf_buf_destroy(mlf_buf* b);
const char* mlf_buf_id(const mlf_buf* b);
uint64_t mlf_buf_capacity(const mlf_buf* b); /* 0 once closed */
void* mlf_buf_host_ptr(const mlf_buf* b);    /* NULL once closed */
int32_t mlf_buf_is_closed(const mlf_buf* b);
int32_t mlf_buf_is_readonly(const mlf_buf* b);
/* Page-lock the mapping and map it for the current CUDA device (cudaHostRegister with the
 * portable+mapped flags, plus read-only for RO mappings). Pages are touched first so that
 * registration does not fault them in one by one. No-op if already registered. The mapping is
 * locked in 512 MiB chunks: mlf_buf_resize of a registered buffer then re-locks only the chunks
 * behind the smaller of the old and new end, and mlf_memcpy_async cuts its transfers at chunk
 * boundaries. Kernels still see one contiguous range (mlf_buf_dev_ptr). */
int32_t mlf_buf_register(mlf_buf* b);
int32_t mlf_buf_unregister(mlf_buf* b);
int32_t mlf_buf_is_registered(const mlf_buf* b);
/* Blocking read of object bytes [offset, offset + nbytes) into device memory, for mappings that are
 * not page-locked (an object opened read-only after a restart cannot be): CPU threads pread() the
 * file into a ring of page-locked slots while copy engines carry the previous chunks. Reading
 * through the descriptor avoids faulting the whole object into the mapping. `nthreads` 0 = half
 * the cores. */
int32_t mlf_buf_read_to_device(const mlf_buf* b, uint64_t offset, void* dev_ptr, uint64_t nbytes, int32_t nthreads);
/* The same read with a second kind of worker beside the pread() threads: one "lock lane" that maps
 * the object's file writable, page-locks `lock_run_mib` MiB of it at a time (cudaHostRegister), lets
 * a copy engine read that piece in place, and unlocks it, one piece ahead of the previous piece's
 * transfer. Both kinds of worker draw from the same range (the threads from its front, the lane
 * from its back) until they meet, so the split follows their speeds. Page-locking moves several
 * times more bytes per CPU core than pread(), but the driver serialises it within a process, so
 * there is one lane; it pays off where the cores, not the host link, bound a restore (several
 * ranks restoring at once on one host). Needs write permission on the file (nothing is written);
 * without it, or if locking fails, the threads move everything. lock_run_mib = 0 is
 * mlf_buf_read_to_device. nthreads < 0 makes the lane work alone (the threads only move what it
 * leaves behind when it cannot run). Same reference counterpart: the loader's per-tensor host reads
 * (core/checkpoint_loader.py:177-219). */
int32_t mlf_buf_read_to_device_hybrid(const mlf_buf* b, uint64_t offset, void* dev_ptr, uint64_t nbytes, int32_t nthreads,
                                      int32_t lock_run_mib);
/* Bytes the lock lane moved during the most recent read in this process (0 if it did not run). */
uint64_t mlf_last_lock_lane_bytes(void);
/* Device-visible address of byte 0 of the mapping (requires registration). */
int32_t mlf_buf_dev_ptr(const mlf_buf* b, void** out);

/* ------------------------------------------------------------------ copy plans
 * Replace the per-tensor host copies on the save and restore paths:
 *   save    `_save_tensor_optimized`: header write + `dest.copy_(tensor)` into the mapping
 *           (core/checkpoint_saver.py:764-800, loop at :667-698)
 *   restore `read_tensor` + `narrow_tensor_by_index` + `target.copy_`
 *           (core/checkpoint_loader.py:177-219, :331-336)
 * A plan is a list of N-d box copies between tensors and one "image": the byte range of a
 * checkpoint object (or its data section). It is built and uploaded once, then launched as ONE
 * kernel per object as often as needed (the tensors of a training job keep their addresses). */
#define MLF_MAX_DIMS 8

#define MLF_PACK 0   /* tensors -> image */
#define MLF_UNPACK 1 /* image -> tensors */

typedef struct mlf_copy_desc {
  uint64_t tensor_ptr;  /* device address of the tensor element with all indices 0 */
  uint64_t image_off;   /* byte offset, in the image, of the box element with all indices 0;
                           any byte alignment is allowed */
  uint32_t elem_size;   /* bytes per element: 1, 2, 4, 8 or 16 */
  uint32_t ndim;        /* 0..MLF_MAX_DIMS; 0 means a single element */
  int64_t shape[MLF_MAX_DIMS];          /* extent of the box per dimension */
  int64_t tensor_stride[MLF_MAX_DIMS];  /* in elements; any non-negative value (views, expands) */
  int64_t image_stride[MLF_MAX_DIMS];   /* in elements; C order of the stored tensor */
} mlf_copy_desc;

typedef struct mlf_plan mlf_plan;

/* Validates and canonicalises the descriptors (drops unit dims, merges mergeable ones, classifies
 * each box as flat / rows / transposed / generic), cuts them into tiles and uploads the tables to
 * the current device. `direction` is MLF_PACK or MLF_UNPACK. */
int32_t mlf_plan_create(const mlf_copy_desc* descs, uint64_t n, int32_t direction, mlf_plan** out);
void mlf_plan_destroy(mlf_plan* p);
/* One past the highest image byte any descriptor touches. */
uint64_t mlf_plan_image_extent(const mlf_plan* p);
/* Sum over descriptors of elements * elem_size. */
uint64_t mlf_plan_payload_bytes(const mlf_plan* p);
uint64_t mlf_plan_num_tiles(const mlf_plan* p);
/* Launches the plan's single kernel on `stream` (a cudaStream_t; NULL = default stream).
 * `image_base` is a device-visible address (HBM, or a registered host mapping) and
 * `image_capacity` the bytes valid behind it: the launch is refused with MLF_ERR_BOUNDS if the
 * plan's extent exceeds it. `max_ctas` limits the grid (0 = one wave sized from the SM count).
 * Launches of ONE plan must not overlap on the GPU (they share the plan's status word and tile
 * counter): order them on one stream or wait for the previous one. */
int32_t mlf_plan_launch(mlf_plan* p, void* image_base, uint64_t image_capacity, void* stream, int32_t max_ctas);
/* After the stream has been synchronised: 0, or the MLF_ERR_* a kernel recorded. Clears it. */
int32_t mlf_plan_status(mlf_plan* p);
/* Gather-pack for callers that cannot obtain device memory: the same kernel as a MLF_PACK plan,
 * with its tables in a fixed array inside the library instead of freshly allocated memory.
 * (No counterpart in the reference implementation, which never touches device memory.)
 *
 * Who needs it: a save that has to run when the process cannot get another byte of HBM, typically
 * an emergency checkpoint right after an out-of-memory error, or any trainer whose own caching
 * allocator has claimed the whole device, so that the cudaMalloc inside mlf_plan_create would
 * fail. This call allocates nothing: no cudaMalloc, cudaFree or other allocating routine, on
 * the device or through a framework. The caller passes inputs (descriptors, tensors) and the
 * output image as for a plan.
 *
 * Limit: at most MLF_NOALLOC_MAX_DESCS descriptors per call; more is refused with
 * MLF_ERR_TOO_LARGE. The array (about 250 KiB) is held by every GPU that loads the library,
 * until the process exits.
 *
 * The first call on a device, with that device current, looks up the array's device address;
 * make that first call outside any stream capture. Better still, make one small real call (a
 * single descriptor) per device at start-up: it brings the library's module, the array and the
 * kernel onto the device while memory is still to be had, which a later call in a tight spot
 * would otherwise have to do itself. All calls on a device share the one array, and it keeps the
 * last call's tables: two calls whose kernels can overlap on the GPU (different streams, or
 * several threads) race on it, so finish one (or order them on one stream) before starting the
 * next. Do not call it while `stream` is being captured: the tables are uploaded from host
 * arrays that the next call overwrites. The kernel runs asynchronously on `stream`, but the call
 * itself may wait for work queued earlier on that stream (the upload is from pageable memory). */
#define MLF_NOALLOC_MAX_DESCS 1024
int32_t mlf_pack_noalloc(const mlf_copy_desc* descs, uint64_t n, void* image_base, uint64_t image_capacity, void* stream);
/* Kernel launches issued by this library since load (for launch accounting in benchmarks). */
uint64_t mlf_launch_count(void);
/* Self-test of the kernels' bounded waits (no counterpart in the reference implementation): one
 * thread waits on a barrier that nothing will complete, gives up after `budget_ns` (at most 100 ms)
 * and records MLF_ERR_TIMEOUT in a status word, exactly as the plan kernels do when a bulk copy
 * does not arrive. Returns MLF_ERR_TIMEOUT when the wait gave up as designed, MLF_OK if it did
 * not. Blocking; the context stays usable afterwards. */
int32_t mlf_selftest_wait_timeout(uint64_t budget_ns, void* stream);

/* ------------------------------------------------------------------ bulk movers
 * Replace the byte movers around the object: the staging copy
 * `tensor.to("cpu")` (adapter/pytorch/memory_storage_writer.py:211-233) and the replication
 * transport `TransferService::AsyncPut` / `ExecutePutTask` / `HandleDataReceive`
 * (replication/transfer_service/transfer_service.cpp:292-332, 632-690, 702-780) for peers that
 * sit in the same NVLink domain. */
#define MLF_COPY_D2H 0
#define MLF_COPY_H2D 1
#define MLF_COPY_D2D 2
/* cudaMemcpyAsync on `stream` (copy-engine DMA). Host memory should be registered. */
int32_t mlf_memcpy_async(void* dst, const void* src, uint64_t nbytes, int32_t kind, void* stream);
/* Blocking transfer between device memory and host memory that is NOT registered with CUDA (for
 * example the read-only mapping of an object opened after a restart). `nthreads` CPU threads
 * (0 = half the cores) move 16 MiB chunks through a ring of page-locked slots while copy engines
 * carry the previous chunks, so the transfer runs at the slower of host memcpy and the host link
 * instead of the driver's pageable path. to_device = 1: host -> device, 0: device -> host.
 * The device range must not be in use by other work while the call runs. */
int32_t mlf_bounce_copy(void* dev_ptr, void* host_ptr, uint64_t nbytes, int32_t to_device, int32_t nthreads);
/* Grid-sized 16-byte vector copy kernel between two device-visible addresses (own HBM, a peer
 * GPU's memory opened through IPC or peer access, or registered host memory). Handles any
 * alignment and size. Used for the NVLink replication hop and as the calibration copy. */
int32_t mlf_copy_kernel_launch(void* dst, const void* src, uint64_t nbytes, void* stream, int32_t max_ctas);

/* Device memory owned by the library (plain cudaMalloc so that IPC handles cover it). */
int32_t mlf_dev_alloc(uint64_t nbytes, void** out);
int32_t mlf_dev_free(void* p);
/* Pinned host scratch (cudaHostAlloc), used for blobs and small uploads. */
int32_t mlf_host_alloc(uint64_t nbytes, void** out);
int32_t mlf_host_free(void* p);
/* CUDA IPC: export an allocation made by mlf_dev_alloc / open one exported by another process. */
#define MLF_IPC_HANDLE_BYTES 64
int32_t mlf_ipc_export(void* dev_ptr, uint8_t handle_out[MLF_IPC_HANDLE_BYTES]);
int32_t mlf_ipc_open(const uint8_t handle[MLF_IPC_HANDLE_BYTES], void** out);
int32_t mlf_ipc_close(void* p);
/* Enable direct access from the current device to `peer_device` (same process). */
int32_t mlf_enable_peer_access(int32_t peer_device);

/* ------------------------------------------------------------------ streams and events
 * The "safe to mutate" signal of an overlapped save: record an event after the pack kernel and
 * make the optimizer's stream wait on it. */
int32_t mlf_set_device(int32_t device);
int32_t mlf_get_device(int32_t* device);
int32_t mlf_device_sm_count(int32_t* out);
int32_t mlf_stream_create(void** out);
int32_t mlf_stream_destroy(void* stream);
int32_t mlf_stream_sync(void* stream);
int32_t mlf_stream_wait_event(void* stream, void* event);
int32_t mlf_event_create(void** out);
int32_t mlf_event_destroy(void* event);
int32_t mlf_event_record(void* event, void* stream);
int32_t mlf_event_sync(void* event);
/* 1 if complete, 0 if still pending, negative on error. */
int32_t mlf_event_query(void* event);
int32_t mlf_event_elapsed_ms(void* start, void* stop, float* ms);

#ifdef __cplusplus
}
#endif
#endif /* MLF_B200_H_ */
