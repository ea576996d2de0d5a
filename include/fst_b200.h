/*
 * fst_b200.h -- C ABI of libfst_b200.so, the native layer of the B200 safetensors loader.
 *
 * This library stands where upstream fastsafetensors has its pybind11 module
 * `fastsafetensors.cpp` (fastsafetensors/cpp/ext.cpp, ext.hpp, cpp.pyi).  Each entry point
 * below names the upstream interface it replaces.  The boundary is plain C: integer status
 * codes, addresses and sizes as 64-bit integers, caller-owned buffers with explicit lengths
 * that are bounds-checked before anything is launched, no C++ or torch types, no exceptions.
 *
 * Conventions
 *   - every function that can fail returns 0 on success and a negative FST_E* code on
 *     failure; fst_last_error() then returns a text for the calling thread;
 *   - "device address" means an address valid on the CUDA device that is current in the
 *     calling thread (or, for readers, the device given at creation);
 *   - `stream` is a cudaStream_t passed as an integer (0 = the legacy default stream);
 *     kernels are only enqueued, never synchronised, unless stated otherwise;
 *   - a library built without a usable CUDA driver still loads: host-side entry points
 *     work, device entry points return FST_ENOCUDA.  Nothing here silently substitutes a
 *     host path for a device path.
 */
#ifndef FST_B200_H
#define FST_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library itself is built with hidden visibility */
#endif

#define FST_B200_ABI_VERSION 2

/* status codes */
#define FST_OK 0
#define FST_EINVAL (-1)   /* bad argument (null pointer, zero handle, size mismatch)      */
#define FST_ERANGE (-2)   /* offset + length exceeds the buffer length the caller stated */
#define FST_ENOCUDA (-3)  /* no CUDA device / driver; device entry point refused          */
#define FST_ECUDA (-4)    /* a CUDA runtime call failed; see fst_last_error()             */
#define FST_EIO (-5)      /* open/pread failed or hit end of file early                   */
#define FST_ETIMEOUT (-6) /* a bounded wait ran out                                      */
#define FST_ENOMEM (-7)   /* host or device allocation failed                            */
#define FST_ELIMIT (-8)   /* request larger than a fixed capacity of the entry point     */
#define FST_EGDS (-9)     /* cuFile ("gds") unavailable or failed                        */

/* ------------------------------------------------------------------------------------------
 * Library state, diagnostics, topology
 * ---------------------------------------------------------------------------------------- */

/* ABI version of the loaded library (FST_B200_ABI_VERSION at build time). */
int fst_abi_version(void);

/* Text of the last error raised on the calling thread ("" if none).  Never NULL. */
const char *fst_last_error(void);

/* Number of CUDA devices visible, 0 when there is no driver or no device.
 * Replaces is_cuda_found() (cpp.pyi; ext.cpp:278-389 decides it by dlopen of libcudart). */
int fst_cuda_device_count(void);

/* Per-call debug lines on stdout on/off.  Replaces set_debug_log() (ext.cpp:480-484). */
void fst_set_debug(int on);

/* PCI bus id ("0000:d1:00.0") of a device into out[0..n).
 * Replaces get_device_pci_bus() (ext.cpp:508-523). */
int fst_device_pci_bus(int device, char *out, int n);

/* NUMA node of a device from sysfs, -1 if unknown.
 * Replaces get_device_numa_node() (fastsafetensors/common.py:40-51). */
int fst_device_numa_node(int device);

/* Bind the calling thread (and threads it creates later) to the CPUs of a NUMA node and
 * prefer that node for new pages, so that the pinned ring is allocated next to the GPU.
 * Replaces set_numa_node() -> numa_run_on_node() (ext.cpp:525-533); libnuma is not needed. */
int fst_pin_numa(int node);

/* Page-aligned (4096) host allocation and release.
 * Replaces cpu_malloc()/cpu_free() (ext.cpp:542-557). */
uint64_t fst_host_alloc(uint64_t nbytes);
void fst_host_free(uint64_t addr);

/* Plain device allocation and release on the current device (cudaMalloc / cudaFree); 0 on
 * failure.  Replaces gpu_malloc()/gpu_free() (ext.cpp:559-569).  The loader itself does not use
 * them (its images are torch allocations); they exist for callers of upstream's module API. */
uint64_t fst_device_alloc(uint64_t nbytes);
void fst_device_free(uint64_t addr);

/* cudaMemcpyAsync host -> device of nbytes on the legacy default stream; returns the CUDA error
 * code (0 = success), or FST_ENOCUDA.  Replaces memcpy_h2d_async() (ext.cpp:959-971). */
int fst_memcpy_h2d_async(uint64_t dst, uint64_t src, uint64_t nbytes);

/* Copy nbytes of HOST memory at addr into out.  Replaces read_buffer() (ext.cpp:535-540). */
int fst_read_host(uint64_t addr, uint64_t nbytes, void *out);

/* I/O alignment of the direct-I/O window (4096).  Replaces get_alignment_size(). */
int fst_io_alignment(void);

/* Counters.  `bounce_buffer_bytes` is upstream's cpp_metrics.bounce_buffer_bytes
 * (ext.hpp:256-258, ext.cpp:744,788): pinned ring bytes currently allocated; it returns to
 * zero when every reader is destroyed.  The rest are cumulative since load. */
typedef struct fst_metrics {
    uint64_t bounce_buffer_bytes;   /* pinned host ring bytes alive now                     */
    uint64_t staging_device_bytes;  /* device staging ring bytes alive now                  */
    uint64_t bytes_read;            /* bytes returned by pread / cuFileRead                 */
    uint64_t bytes_h2d;             /* bytes handed to cudaMemcpyAsync host->device         */
    uint64_t bytes_realigned;       /* bytes moved by the realign kernel                    */
    uint64_t bytes_gathered;        /* payload bytes moved by the gather kernel             */
    uint64_t kernel_launches;       /* launches of this library's own kernels               */
    uint64_t direct_io_requests;    /* read requests served with O_DIRECT                   */
    uint64_t buffered_io_requests;  /* read requests served through the page cache          */
    uint64_t read_ns;               /* summed wall time workers spent inside pread          */
    uint64_t reserved[6];
} fst_metrics_t;
int fst_get_metrics(fst_metrics_t *out);

/* ------------------------------------------------------------------------------------------
 * Reader: file bytes -> pinned ring -> destination buffer (HBM or host)
 *
 * Replaces nogds_file_reader (ext.hpp:155-185, ext.cpp:648-806: one std::thread per request,
 * buffered pread into a per-thread bounce chunk, synchronous cudaMemcpy) and the read side of
 * gds_file_reader / gds_file_handle (ext.cpp:808-950).
 *
 * A reader owns `threads` worker threads, a ring of page-aligned pinned slots
 * (threads * slots_per_thread slots of slot_bytes) and, for a device destination,
 * `copy_streams` CUDA streams plus a device staging ring used only when a file's data
 * section is not 16-byte congruent with its destination.  A request is cut into slot-sized,
 * 4096-aligned file windows; a worker reads a window (O_DIRECT when the file is not in the
 * page cache, buffered when it is), then enqueues cudaMemcpyAsync to the destination and
 * moves on to its other slot, so the read of window k+1 overlaps the DMA of window k.  When
 * source and destination are not 16-byte congruent the DMA lands the whole window in the
 * device staging slot and the realign kernel shifts it into place.
 * ---------------------------------------------------------------------------------------- */

#define FST_IO_AUTO 0     /* direct I/O unless most of the file is resident in the page cache */
#define FST_IO_DIRECT 1   /* O_DIRECT; falls back to buffered if the filesystem refuses it   */
#define FST_IO_BUFFERED 2 /* plain pread through the page cache                              */
#define FST_IO_CUFILE 3   /* cuFileRead into the registered device staging ring (device dst only);
                             FST_EGDS, with "gds" in the error text, when cuFile cannot be used:
                             no libcufile, or no nvidia-fs module (checked BEFORE the cuFile
                             driver is opened; its compatibility mode is never entered)          */

typedef struct fst_reader_config {
    int32_t device;           /* CUDA device of destinations; -1: destinations are host memory */
    int32_t threads;          /* worker threads (upstream max_threads)                         */
    int32_t slots_per_thread; /* ring depth per worker, >= 1 (2 = double buffering)            */
    int32_t io_mode;          /* FST_IO_*                                                      */
    uint64_t slot_bytes;      /* bytes per slot, rounded up to a multiple of 4096              */
    int32_t copy_streams;     /* H2D streams shared by the workers, >= 1                       */
    int32_t numa_node;        /* bind workers and ring to this node, -1: leave as is           */
    int32_t plain_dma_only;   /* 1: never use the realign kernel, DMA to unaligned addresses   */
    int32_t reserved[7];
} fst_reader_config_t;

/* Create a reader.  Nothing is allocated yet: streams, events and threads come with the first
 * submit, and every worker pins its own slots when it gets its first window (upstream pins its
 * whole bounce buffer at the first submit, ext.cpp:735-751).  Pinned bytes are counted in
 * fst_metrics.bounce_buffer_bytes. */
int fst_reader_create(const fst_reader_config_t *cfg, uint64_t *reader);

/* Queue the read of file bytes [file_offset, file_offset + nbytes) of `path` into
 * dst[dst_offset, dst_offset + nbytes).  dst_len is the length of the destination buffer;
 * dst_offset + nbytes > dst_len is refused with FST_ERANGE (upstream: _get_raw_pointer,
 * ext.hpp:139-146).  Returns at once; *request receives an id for fst_reader_wait.
 * Replaces nogds_file_reader::submit_read (ext.cpp:726-763) and
 * gds_file_reader::submit_read (ext.cpp:910-934). */
int fst_reader_submit(uint64_t reader, const char *path, uint64_t file_offset, uint64_t nbytes,
                      uint64_t dst, uint64_t dst_len, uint64_t dst_offset, int64_t *request);

/* Order every copy this reader issues from now on behind the work queued so far on `stream`
 * (one event recorded there, waited for by all copy streams).  Call it after allocating a
 * destination from a stream-ordered allocator and before fst_reader_submit: the memory may have
 * belonged to a buffer that kernels already queued on `stream` still read, and the reader's copy
 * streams are otherwise independent of it.  (Upstream needs no such call: its cudaMemcpy on the
 * legacy default stream is ordered behind everything, ext.cpp:700-712.)  No-op for host readers. */
int fst_reader_order_after(uint64_t reader, uint64_t stream);

/* Block until the request's bytes are in the destination (DMA and kernels complete) or
 * timeout_ms passes (< 0: no limit).  *bytes_done receives the bytes delivered.  A failed or
 * short read returns FST_EIO after every window of the request has been drained.  After
 * FST_ETIMEOUT the request is still known: wait for it again with the same id.
 * Replaces nogds_file_reader::wait_read (ext.cpp:765-776) / gds_file_reader::wait_read. */
int fst_reader_wait(uint64_t reader, int64_t request, int64_t timeout_ms, uint64_t *bytes_done);

/* Join the workers, free ring, staging ring and streams.  Replaces ~nogds_file_reader
 * (ext.cpp:778-806). */
int fst_reader_destroy(uint64_t reader);

/* 1 if libcufile.so can be loaded.  Replaces is_cufile_found() (cpp.pyi). */
int fst_cufile_available(void);
/* 1 if GPUDirect Storage proper can work for this device (the nvidia-fs module is loaded), 0 if
 * cuFile could only run in its compatibility mode.  Replaces is_gds_supported() (ext.cpp:444-478). */
int fst_gds_supported(int device);

/* Host-side fault injection for tests: the nth pread from now on (1-based, counted over all
 * workers of this reader) fails with `err` (an errno value), or, if short_bytes >= 0,
 * returns only short_bytes bytes.  nth = 0 disarms.  No GPU fault is involved. */
int fst_reader_inject_fault(uint64_t reader, int64_t nth, int err, int64_t short_bytes);

/* ------------------------------------------------------------------------------------------
 * Kernels (sm_100a)
 * ---------------------------------------------------------------------------------------- */

/* One strided 2-D byte copy: for r in [0, rows): dst[r*dst_pitch ..+row_bytes) =
 * src[r*src_pitch ..+row_bytes).  A dim-0 shard, a dim-1 shard, an N-d shard on any dim and
 * one member of a multi-column concatenation are each one such copy. */
typedef struct fst_copy2d {
    uint64_t src;       /* address of the first source byte      */
    uint64_t dst;       /* address of the first destination byte */
    uint64_t rows;
    uint64_t row_bytes;
    uint64_t src_pitch; /* bytes between source row starts       */
    uint64_t dst_pitch; /* bytes between destination row starts  */
} fst_copy2d_t;

/* Shard gather / pack: run n_ops strided copies in ONE launch on `stream`.
 * Replaces the W `t[slices].contiguous()` launches of LazyTensorFactory.shuffle
 * (tensor_factory.py:168-175) and the per-rank torch.cat of shuffle_multi_cols
 * (tensor_factory.py:240-246).  Any byte alignment of addresses, pitches and widths is
 * accepted; 16-byte congruent rows move as 16-byte vectors, others through a byte-shift path.
 * If src_len (dst_len) is non-zero every op's source (destination) range must lie inside
 * [src_base, src_base+src_len) ([dst_base, dst_base+dst_len)) or FST_ERANGE is returned and
 * nothing is launched.  Ranges of different ops must not overlap in the destination.
 * Up to FST_GATHER_INLINE_OPS ops travel in the kernel's parameters; larger tables are staged
 * through a device workspace owned by the library (allocated on first use, per device). */
#define FST_GATHER_INLINE_OPS 48
int fst_gather(const fst_copy2d_t *ops, uint64_t n_ops, uint64_t src_base, uint64_t src_len,
               uint64_t dst_base, uint64_t dst_len, uint64_t stream);

/* fst_gather with an upper bound on the number of CTAs of each launch (0 = the library's own
 * rule).  The kernel strides over its work, so a small grid only means that each CTA takes more
 * steps.  For copies whose destination is another GPU's memory: a few hundred CTAs keep enough
 * stores in flight to fill NVLink, and leave the rest of the SMs to a second gather (this GPU's
 * own region) running beside it on another stream.  (No counterpart in upstream.) */
int fst_gather_limited(const fst_copy2d_t *ops, uint64_t n_ops, uint64_t src_base, uint64_t src_len,
                       uint64_t dst_base, uint64_t dst_len, uint64_t stream, uint32_t max_ctas);

/* fst_gather for callers that must not allocate.  (No counterpart in upstream: its native
 * layer has no kernels and therefore no kernel workspace.)
 *
 * Who needs it: a loader that runs inside a process whose device memory is already spoken for --
 * an inference server that has handed all free HBM to its KV-cache pool, or a host application
 * that forbids the CUDA allocator after start-up because cudaMalloc/cudaFree synchronise the
 * whole device and would stall the streams that are serving requests.  For such callers the
 * workspace that fst_gather allocates on first use for large op tables can fail or is not
 * allowed at all.
 *
 * This entry point does the same copies with the same kernel but keeps its op table in a fixed
 * array that is part of the library image: a file-scope `static __device__` array of
 * FST_GATHER_STATIC_MAX_OPS records (64 bytes each, 256 KiB), which every GPU that loads the
 * library holds until the process exits.  It calls no cudaMalloc, cudaFree, cudaHostAlloc or any
 * other allocating routine, on the device or on the host.
 *
 *   - n_ops > FST_GATHER_STATIC_MAX_OPS is refused with FST_ELIMIT (split the request).
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current) and keeps it.
 *   - All calls on a device share the one array.  A call overwrites the entries it uses and
 *     never reads beyond them, so nothing needs clearing between calls; but a call must not be
 *     issued while an earlier call on ANOTHER stream may still be running, or the earlier kernel
 *     can read a half-rewritten table.  Calls on one stream are ordered and safe.
 *   - The table is uploaded with cudaMemcpyAsync from ordinary (pageable) host memory, which
 *     returns once the runtime has staged the bytes, so the caller's ops array may be reused
 *     as soon as the call returns.  For such a copy the runtime first waits, on the host, for
 *     the work already queued on `stream`: the calling thread stalls for that long, and other
 *     threads calling fst_gather_static wait behind it (fst_gather callers do not).
 * Arguments, checks and results are those of fst_gather. */
#define FST_GATHER_STATIC_MAX_OPS 4096
int fst_gather_static(const fst_copy2d_t *ops, uint64_t n_ops, uint64_t src_base,
                      uint64_t src_len, uint64_t dst_base, uint64_t dst_len, uint64_t stream);

/* The same copies done by host threads, for buffers in host memory (device "cpu").  This is
 * the loader's CPU mode, not a substitute for fst_gather on device buffers. */
int fst_gather_host(const fst_copy2d_t *ops, uint64_t n_ops, int threads);

/* Realign: out-of-place copy of nbytes from src to dst where the two addresses need not be
 * congruent modulo 16; dst is written with 16-byte stores, src is read with 16-byte loads and
 * re-packed with funnel shifts.  The ranges must not overlap.
 * Replaces gds_device_buffer::memmove (ext.cpp:606-645: two cudaMemcpy through a 1 GiB
 * temporary, i.e. 4x the payload in HBM traffic) as used by GdsFileCopier.wait_io
 * (copier/gds.py:138-159). */
int fst_realign(uint64_t dst, uint64_t src, uint64_t nbytes, uint64_t stream);

/* Narrowing conversion at load time: many tensors in ONE launch, out of place.
 * Replaces the per-tensor `t.to(dtype)` + `copy_` of SafeTensorsMetadata.get_tensors
 * (common.py:355-375, two torch kernels and a temporary per tensor).  Floating-point types
 * only; the destination must not be wider than the source; rounding is round-to-nearest-even
 * through float (what `torch.Tensor.to` does on a CUDA device); ranges must not overlap and
 * addresses must be aligned to their element size. */
#define FST_DT_F64 0
#define FST_DT_F32 1
#define FST_DT_F16 2
#define FST_DT_BF16 3
typedef struct fst_convert_op {
    uint64_t src;
    uint64_t dst;
    uint64_t n_elements;
    int32_t src_dtype; /* FST_DT_* */
    int32_t dst_dtype; /* FST_DT_F32, FST_DT_F16 or FST_DT_BF16 */
} fst_convert_op_t;
int fst_convert(const fst_convert_op_t *ops, uint64_t n_ops, uint64_t stream);

/* ------------------------------------------------------------------------------------------
 * Peer arenas: receive buffers that the other ranks of one machine can write into
 *
 * Replaces the transport half of LazyTensorFactory.shuffle / shuffle_multi_cols
 * (tensor_factory.py:186,258 -> frameworks/_torch.py:151-178: one NCCL scatter and a device
 * synchronisation per tensor).  Every rank creates an arena sized for what it will receive,
 * exports a 64-byte handle, and opens the handles of its peers; the owner of a file then gives
 * fst_gather destination addresses inside its peers' arenas, so the pack and the transfer are
 * one kernel: shards leave the owner's HBM once and land in the consumer's HBM over NVLink.
 * A barrier after the launch (any small collective on the same stream) tells a rank that all
 * its peers' kernels have finished.  Importers must close their mapping before the exporter
 * destroys the arena.
 * ---------------------------------------------------------------------------------------- */
#define FST_ARENA_HANDLE_BYTES 64

/* cudaMalloc an arena of nbytes on the current device; *arena is its device address. */
int fst_arena_create(uint64_t nbytes, uint64_t *arena);
/* Write the arena's inter-process handle (FST_ARENA_HANDLE_BYTES) into handle. */
int fst_arena_export(uint64_t arena, void *handle, uint64_t handle_bytes);
/* Map a peer's arena into this process; *peer_addr is valid on the current device. */
int fst_arena_open_peer(const void *handle, uint64_t handle_bytes, uint64_t *peer_addr);
int fst_arena_close_peer(uint64_t peer_addr);
int fst_arena_destroy(uint64_t arena);

/* Free the per-device workspaces of fst_gather (they are also freed at process exit). */
int fst_release_workspaces(void);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* FST_B200_H */
