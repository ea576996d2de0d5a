// Reader of libfst_b200.so: file bytes -> ring of pinned slots -> destination (HBM or host).
//
// One reader = a pool of worker threads + a ring of page-aligned slots + (device destinations
// only) a few copy streams and a lazily allocated device staging ring.  A request is cut into
// windows of slot_bytes whose file offsets are multiples of 4096, so the same windows serve
// O_DIRECT and buffered reads.  Each worker owns `slots_per_thread` slots and walks them round
// robin: wait for the slot's previous DMA (event), pread the window, enqueue the DMA, move on.
// With two slots per worker the pread of window k+1 runs while the copy engine moves window k.
//
// Alignment of the DMA.  Let s be the host address of the first valid byte in the slot and d
// its destination address.  If s and d are congruent modulo 16 the valid bytes are copied
// straight to d.  If not (a safetensors header of odd length, say), the 16-byte-aligned
// envelope of the valid bytes is copied to the slot's twin in a device staging ring and the
// realign kernel shifts it to d on the same stream; the copy engine only ever sees 16-byte
// aligned addresses, and the shift costs 2 x payload of HBM traffic instead of a slower DMA.
#include <cuda_runtime.h>
#include <cufile.h>
#include <dlfcn.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <cerrno>
#include <chrono>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_set>
#include <vector>

#include "fst_internal.h"

namespace fst {
namespace {

constexpr uint64_t IO_ALIGN = 4096;

// cuFile entry points, resolved from libcufile.so at run time (the library is optional).
struct CuFileApi {
    CUfileError_t (*DriverOpen)() = nullptr;
    CUfileError_t (*DriverClose)() = nullptr;
    CUfileError_t (*HandleRegister)(CUfileHandle_t *, CUfileDescr_t *) = nullptr;
    void (*HandleDeregister)(CUfileHandle_t) = nullptr;
    CUfileError_t (*BufRegister)(const void *, size_t, int) = nullptr;
    CUfileError_t (*BufDeregister)(const void *) = nullptr;
    ssize_t (*Read)(CUfileHandle_t, void *, size_t, off_t, off_t) = nullptr;
    bool loaded = false;
    bool tried = false;
    bool stand_in = false;  // a test double that needs neither the cuFile driver nor nvidia-fs
    int driver_users = 0;
};
CuFileApi g_cufile;
std::mutex g_cufile_mutex;

// FST_B200_CUFILE_LIB names a library to load in place of libcufile.so.  It is meant for a
// host-side double of the seven entry points (tests run the cuFile code path through one, as
// upstream runs its own through a table of fakes, ext.cpp:126-196).  A library counts as such a
// double only if it also exports the marker symbol `fst_cufile_stand_in`; for anything else the
// nvidia-fs check of cufile_acquire() still applies, so the variable cannot be used to walk the
// real library into a host on which it cannot work.
bool load_cufile_locked() {
    if (g_cufile.tried) return g_cufile.loaded;
    g_cufile.tried = true;
    void *h = nullptr;
    const char *named = std::getenv("FST_B200_CUFILE_LIB");
    if (named && named[0]) {
        h = dlopen(named, RTLD_NOW | RTLD_LOCAL);
    } else {
        for (const char *name : {"libcufile.so.0", "libcufile.so"}) {
            h = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (h) break;
        }
    }
    if (!h) return false;
    auto sym = [&](const char *n) { return dlsym(h, n); };
    g_cufile.stand_in = sym("fst_cufile_stand_in") != nullptr;
    g_cufile.DriverOpen = (decltype(g_cufile.DriverOpen))sym("cuFileDriverOpen");
    g_cufile.DriverClose = (decltype(g_cufile.DriverClose))sym("cuFileDriverClose");
    g_cufile.HandleRegister = (decltype(g_cufile.HandleRegister))sym("cuFileHandleRegister");
    g_cufile.HandleDeregister = (decltype(g_cufile.HandleDeregister))sym("cuFileHandleDeregister");
    g_cufile.BufRegister = (decltype(g_cufile.BufRegister))sym("cuFileBufRegister");
    g_cufile.BufDeregister = (decltype(g_cufile.BufDeregister))sym("cuFileBufDeregister");
    g_cufile.Read = (decltype(g_cufile.Read))sym("cuFileRead");
    g_cufile.loaded = g_cufile.DriverOpen && g_cufile.HandleRegister && g_cufile.HandleDeregister &&
                      g_cufile.BufRegister && g_cufile.BufDeregister && g_cufile.Read;
    return g_cufile.loaded;
}

// Opens the cuFile driver for one more user.  Returns FST_OK or FST_EGDS (error text set).
int cufile_acquire() {
    std::lock_guard<std::mutex> lock(g_cufile_mutex);
    // Without the nvidia-fs module cuFile could only run in its compatibility mode, and on hosts
    // that also lack a udev database cuFileDriverOpen() has been seen never to return.  Such a
    // host gets the error a caller retries on (vLLM looks for "gds" in the text and loads again
    // with nogds=True) instead of a call that may hang; libcufile is not even loaded.
    const char *named = std::getenv("FST_B200_CUFILE_LIB");
    const bool substitute = named && named[0];
    if (!substitute && fst_gds_supported(0) == 0) {
        set_error("gds: the nvidia-fs kernel module is not loaded; cuFile's compatibility mode "
                  "is not used");
        return FST_EGDS;
    }
    if (!load_cufile_locked()) {
        set_error("gds: %s could not be loaded", substitute ? named : "libcufile.so");
        return FST_EGDS;
    }
    if (!g_cufile.stand_in && fst_gds_supported(0) == 0) {  // a named library that is no double
        set_error("gds: the nvidia-fs kernel module is not loaded; cuFile's compatibility mode "
                  "is not used");
        return FST_EGDS;
    }
    if (g_cufile.driver_users == 0) {
        FST_DEBUG("cufile: calling cuFileDriverOpen");
        const CUfileError_t e = g_cufile.DriverOpen();
        FST_DEBUG("cufile: cuFileDriverOpen returned %d", (int)e.err);
        if (e.err != CU_FILE_SUCCESS) {
            set_error("gds: cuFileDriverOpen failed with cuFile error %d", (int)e.err);
            return FST_EGDS;
        }
    }
    ++g_cufile.driver_users;
    return FST_OK;
}

void cufile_release() {
    std::lock_guard<std::mutex> lock(g_cufile_mutex);
    if (g_cufile.driver_users > 0 && --g_cufile.driver_users == 0 && g_cufile.DriverClose)
        g_cufile.DriverClose();
}

inline uint64_t align_down(uint64_t v, uint64_t a) { return v - v % a; }
inline uint64_t align_up(uint64_t v, uint64_t a) { return align_down(v + a - 1, a); }
inline uint64_t now_ns() {
    return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
               std::chrono::steady_clock::now().time_since_epoch())
        .count();
}

// Fraction of the pages of file range [off, off+len) that sit in the page cache, or -1.
// Uses cachestat(2) (Linux >= 6.5), else mincore(2) on a temporary mapping.
double cached_fraction(int fd, uint64_t off, uint64_t len) {
    if (len == 0) return 0.0;
    const uint64_t pages = (len + IO_ALIGN - 1) / IO_ALIGN;
#ifndef SYS_cachestat
#define SYS_cachestat 451
#endif
    struct {
        uint64_t off, len;
    } range = {off, len};
    struct {
        uint64_t nr_cache, nr_dirty, nr_writeback, nr_evicted, nr_recently_evicted;
    } cs = {};
    if (syscall(SYS_cachestat, fd, &range, &cs, 0u) == 0) return (double)cs.nr_cache / (double)pages;
    const uint64_t a = align_down(off, IO_ALIGN);
    const uint64_t mlen = off + len - a;
    void *m = mmap(nullptr, mlen, PROT_READ, MAP_SHARED, fd, (off_t)a);
    if (m == MAP_FAILED) return -1.0;
    const uint64_t npg = (mlen + IO_ALIGN - 1) / IO_ALIGN;
    // sample at most 4096 evenly spaced pages through page-sized mincore calls
    const uint64_t samples = npg < 4096 ? npg : 4096;
    uint64_t hit = 0;
    for (uint64_t i = 0; i < samples; ++i) {
        unsigned char v = 0;
        const uint64_t pg = npg * i / samples;
        if (mincore((char *)m + pg * IO_ALIGN, IO_ALIGN, &v) == 0 && (v & 1)) ++hit;
    }
    munmap(m, mlen);
    return (double)hit / (double)samples;
}

struct Request {
    int64_t id = 0;
    int fd = -1;
    bool direct = false;
    bool cufile = false;
    CUfileHandle_t cf_handle = nullptr;
    uint64_t remaining = 0;   // windows not yet handed to the copy engine / destination
    uint64_t bytes_done = 0;
    std::atomic<int> status{FST_OK};  // written under the reader's mutex; workers peek at it
                                       // without the lock to skip the I/O of a failed request
    std::string error;
};

struct Task {
    std::shared_ptr<Request> req;
    uint64_t win_off = 0;    // file offset of the window (multiple of 4096)
    uint64_t win_len = 0;    // bytes to read (multiple of 4096; may extend past end of file)
    uint64_t valid_off = 0;  // file offset of the first byte wanted
    uint64_t valid_len = 0;  // bytes wanted from this window
    uint64_t dst = 0;        // destination address of the first wanted byte
};

struct Slot {
    unsigned char *host = nullptr;
    unsigned char *stage = nullptr;  // device twin, allocated when first needed
    cudaEvent_t done = nullptr;
    bool pending = false;
};

class Reader {
  public:
    explicit Reader(const fst_reader_config_t &c) : cfg_(c) {}
    ~Reader() { shutdown(); }

    int submit(const char *path, uint64_t file_off, uint64_t nbytes, uint64_t dst,
               uint64_t dst_len, uint64_t dst_off, int64_t *out_id);
    int wait(int64_t id, int64_t timeout_ms, uint64_t *bytes_done);
    void inject(int64_t nth, int err, int64_t short_bytes) {
        std::lock_guard<std::mutex> lock(mu_);
        fault_nth_ = nth;
        fault_err_ = err;
        fault_short_ = short_bytes;
        reads_seen_ = 0;
        fault_armed_.store(nth > 0, std::memory_order_release);
    }
    int order_after(uint64_t stream);
    void shutdown();

  private:
    int start();  // streams, events, threads (first submit)
    int ensure_worker_ring(int worker_index);
    int ensure_stage_ring();
    void worker(int index);
    void run_task(const Task &t, Slot &slot, int worker_index);
    void run_cufile_task(const Task &t, Slot &slot, int worker_index);
    ssize_t do_pread(int fd, void *buf, size_t len, off_t off);
    void finish(const Task &t, int status, const std::string &err, uint64_t bytes);

    fst_reader_config_t cfg_;
    bool started_ = false;
    bool stopping_ = false;
    std::vector<unsigned char *> worker_ring_;  // one block of slots per worker, allocated by it
    std::atomic<uint64_t> ring_bytes_{0};
    bool ring_pinned_ = false;
    bool cufile_open_ = false;       // this reader holds a reference on the cuFile driver
    bool stage_registered_ = false;  // the staging ring is registered with cuFile
    uint64_t stage_bytes_ = 0;
    unsigned char *stage_ring_ = nullptr;
    std::vector<Slot> slots_;
    std::vector<cudaStream_t> streams_;
    std::vector<std::thread> threads_;

    std::mutex ring_mu_;
    std::mutex mu_;
    std::condition_variable work_cv_;   // workers wait for tasks
    std::condition_variable done_cv_;   // waiters wait for requests
    std::deque<Task> queue_;
    std::map<int64_t, std::shared_ptr<Request>> requests_;
    int64_t next_id_ = 1;
    int64_t fault_nth_ = 0, fault_short_ = -1, reads_seen_ = 0;
    int fault_err_ = 0;
    std::atomic<bool> fault_armed_{false};
    cudaEvent_t order_event_ = nullptr;  // see order_after
};

// Creates what the first submit needs.  Every resource is created at most once: a call that
// failed halfway (a stream or an event could not be made) is picked up where it stopped by the
// next call instead of creating the earlier resources a second time.
int Reader::start() {
    if (started_) return FST_OK;
    const int nslots = cfg_.threads * cfg_.slots_per_thread;
    if (cfg_.device >= 0) {
        cudaError_t e = cudaSetDevice(cfg_.device);
        if (e != cudaSuccess) {
            set_error("reader: cudaSetDevice(%d) failed: %s", cfg_.device, cudaGetErrorString(e));
            return FST_ECUDA;
        }
        while ((int)streams_.size() < cfg_.copy_streams) {
            cudaStream_t s = nullptr;
            e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
            if (e != cudaSuccess) {
                (void)cudaGetLastError();
                set_error("reader: cudaStreamCreate failed: %s", cudaGetErrorString(e));
                return FST_ECUDA;
            }
            streams_.push_back(s);
        }
        if (order_event_ == nullptr) {
            e = cudaEventCreateWithFlags(&order_event_, cudaEventDisableTiming);
            if (e != cudaSuccess) {
                (void)cudaGetLastError();
                order_event_ = nullptr;
                set_error("reader: cudaEventCreate failed: %s", cudaGetErrorString(e));
                return FST_ECUDA;
            }
        }
    }
    if ((int)slots_.size() != nslots) slots_.resize(nslots);
    if (cfg_.device >= 0) {
        for (int i = 0; i < nslots; ++i) {
            if (slots_[i].done != nullptr) continue;
            const cudaError_t e = cudaEventCreateWithFlags(&slots_[i].done, cudaEventDisableTiming);
            if (e != cudaSuccess) {
                (void)cudaGetLastError();
                slots_[i].done = nullptr;
                set_error("reader: cudaEventCreate failed: %s", cudaGetErrorString(e));
                return FST_ECUDA;
            }
        }
        if (cfg_.io_mode == FST_IO_CUFILE) {
            // cuFile lands file windows in the device staging ring directly; no host ring
            if (!cufile_open_) {
                const int rc = cufile_acquire();
                if (rc != FST_OK) return rc;
                cufile_open_ = true;
            }
            const int rc = ensure_stage_ring();
            if (rc != FST_OK) {
                set_error("gds: device staging ring allocation failed");
                return rc;
            }
            if (!stage_registered_) {
                FST_DEBUG("cufile: registering the staging ring");
                const CUfileError_t e2 = g_cufile.BufRegister(stage_ring_, stage_bytes_, 0);
                stage_registered_ = e2.err == CU_FILE_SUCCESS;  // unregistered buffers still work
                FST_DEBUG("reader: cuFile staging ring of %llu bytes, registered=%d",
                          (unsigned long long)stage_bytes_, (int)stage_registered_);
            }
        }
    }
    worker_ring_.assign(cfg_.threads, nullptr);
    ring_pinned_ = cfg_.device >= 0;
    started_ = true;
    for (int i = 0; i < cfg_.threads; ++i) threads_.emplace_back(&Reader::worker, this, i);
    return FST_OK;
}

// Orders everything this reader copies from now on behind the work queued so far on `stream`.
// A destination buffer that comes from a stream-ordered allocator (torch's caching allocator)
// may still be read by kernels queued on the allocating stream under its previous owner; the
// reader writes through its own non-blocking copy streams, which know nothing of that stream
// unless told.  One event is recorded on `stream` and every copy stream waits for it.
int Reader::order_after(uint64_t stream) {
    if (cfg_.device < 0) return FST_OK;
    std::lock_guard<std::mutex> lock(mu_);
    const int rc = start();
    if (rc != FST_OK) return rc;
    cudaError_t e = cudaEventRecord(order_event_, (cudaStream_t)stream);
    for (size_t i = 0; e == cudaSuccess && i < streams_.size(); ++i)
        e = cudaStreamWaitEvent(streams_[i], order_event_, 0);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        set_error("reader: ordering the copy streams behind stream %#llx failed: %s",
                  (unsigned long long)stream, cudaGetErrorString(e));
        return FST_ECUDA;
    }
    return FST_OK;
}

// Allocates the device twin of the slot ring in ONE cudaMalloc, the first time a window needs the
// realign kernel (cudaMalloc synchronises the device: one call, not one per slot).
int Reader::ensure_stage_ring() {
    std::lock_guard<std::mutex> lock(ring_mu_);
    if (stage_ring_ != nullptr) return FST_OK;
    const uint64_t bytes = (uint64_t)slots_.size() * cfg_.slot_bytes;
    const cudaError_t e = cudaMalloc((void **)&stage_ring_, bytes);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        stage_ring_ = nullptr;
        return FST_ENOMEM;
    }
    stage_bytes_ = bytes;
    g_counters.staging_device_bytes.fetch_add(bytes);
    for (size_t i = 0; i < slots_.size(); ++i) slots_[i].stage = stage_ring_ + i * cfg_.slot_bytes;
    return FST_OK;
}

// Allocates the slots of one worker, on that worker's thread, the first time it needs them.
// Pinning host memory costs about half a millisecond per MiB; done by all workers at once it
// overlaps with the first reads instead of delaying them by the whole ring's worth.  A host
// destination read through the page cache is filled in place and never needs slots.
int Reader::ensure_worker_ring(int w) {
    if (worker_ring_[w] != nullptr) return FST_OK;
    const uint64_t bytes = (uint64_t)cfg_.slots_per_thread * cfg_.slot_bytes;
    unsigned char *block = nullptr;
    if (cfg_.device >= 0) {
        const cudaError_t e = cudaHostAlloc((void **)&block, bytes, cudaHostAllocDefault);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            return FST_ENOMEM;
        }
    } else {
        void *p = nullptr;
        if (posix_memalign(&p, IO_ALIGN, bytes) != 0) return FST_ENOMEM;
        block = (unsigned char *)p;
    }
    worker_ring_[w] = block;
    ring_bytes_.fetch_add(bytes);
    g_counters.bounce_buffer_bytes.fetch_add(bytes);
    for (int i = 0; i < cfg_.slots_per_thread; ++i)
        slots_[(size_t)w * cfg_.slots_per_thread + i].host = block + (uint64_t)i * cfg_.slot_bytes;
    FST_DEBUG("reader: worker %d: %d slots of %llu bytes (%s)", w, cfg_.slots_per_thread,
              (unsigned long long)cfg_.slot_bytes, ring_pinned_ ? "pinned" : "pageable");
    return FST_OK;
}

void Reader::shutdown() {
    {
        std::lock_guard<std::mutex> lock(mu_);
        stopping_ = true;
    }
    work_cv_.notify_all();
    for (auto &t : threads_)
        if (t.joinable()) t.join();
    threads_.clear();
    if (cfg_.device >= 0 && started_) cudaSetDevice(cfg_.device);
    for (auto &s : streams_) {
        cudaStreamSynchronize(s);
        cudaStreamDestroy(s);
    }
    streams_.clear();
    for (auto &s : slots_)
        if (s.done) cudaEventDestroy(s.done);
    slots_.clear();
    if (order_event_) cudaEventDestroy(order_event_);
    order_event_ = nullptr;
    if (stage_registered_) g_cufile.BufDeregister(stage_ring_);
    stage_registered_ = false;
    if (stage_ring_) cudaFree(stage_ring_);
    stage_ring_ = nullptr;
    if (cufile_open_) cufile_release();
    cufile_open_ = false;
    if (stage_bytes_) g_counters.staging_device_bytes.fetch_sub(stage_bytes_);
    stage_bytes_ = 0;
    for (auto &block : worker_ring_) {
        if (block == nullptr) continue;
        if (ring_pinned_) cudaFreeHost(block);
        else std::free(block);
        block = nullptr;
    }
    g_counters.bounce_buffer_bytes.fetch_sub(ring_bytes_.exchange(0));
    for (auto &kv : requests_) {
        if (kv.second->cf_handle) g_cufile.HandleDeregister(kv.second->cf_handle);
        kv.second->cf_handle = nullptr;
        if (kv.second->fd >= 0) {
            close(kv.second->fd);
            kv.second->fd = -1;
        }
    }
    requests_.clear();
}

int Reader::submit(const char *path, uint64_t file_off, uint64_t nbytes, uint64_t dst,
                   uint64_t dst_len, uint64_t dst_off, int64_t *out_id) {
    if (dst_off > dst_len || nbytes > dst_len - dst_off) {
        set_error("reader: out of bound access: buffer length=%llu, request offset=%llu, "
                  "request length=%llu", (unsigned long long)dst_len,
                  (unsigned long long)dst_off, (unsigned long long)nbytes);
        return FST_ERANGE;
    }
    std::unique_lock<std::mutex> lock(mu_);
    int rc = start();
    if (rc != FST_OK) return rc;

    auto req = std::make_shared<Request>();
    req->id = next_id_++;
    int flags = O_RDONLY | O_CLOEXEC;
    int fd = -1;
    bool direct = cfg_.io_mode != FST_IO_BUFFERED;
    const bool cufile = cfg_.io_mode == FST_IO_CUFILE;
    if (cufile && cfg_.device < 0) {
        set_error("gds: cuFile reads need a device destination");
        return FST_EGDS;
    }
    if (cfg_.io_mode == FST_IO_AUTO) {
        fd = open(path, flags);
        if (fd >= 0) {
            const double frac = cached_fraction(fd, file_off, nbytes);
            direct = !(frac >= 0.9);
            FST_DEBUG("reader: %s: %.0f%% of the range is in the page cache -> %s", path,
                      frac * 100.0, direct ? "direct" : "buffered");
            if (direct) {
                close(fd);
                fd = -1;
            }
        }
    }
    if (fd < 0 && direct) {
        fd = open(path, flags | O_DIRECT);
        if (fd < 0 && errno == EINVAL) direct = false;  // filesystem without O_DIRECT (tmpfs)
    }
    if (fd < 0 && !direct) fd = open(path, flags);
    if (fd < 0) {
        set_error("reader: open(%s) failed: %s", path, std::strerror(errno));
        return FST_EIO;
    }
    struct stat st;
    if (fstat(fd, &st) != 0 || file_off + nbytes > (uint64_t)st.st_size) {
        set_error("reader: %s: request [%llu,%llu) extends past the end of the file (%lld bytes)",
                  path, (unsigned long long)file_off, (unsigned long long)(file_off + nbytes),
                  (long long)st.st_size);
        close(fd);
        return FST_EIO;
    }
    req->fd = fd;
    req->direct = direct;
    if (cufile) {
        CUfileDescr_t descr;
        std::memset(&descr, 0, sizeof(descr));
        descr.handle.fd = fd;
        descr.type = CU_FILE_HANDLE_TYPE_OPAQUE_FD;
        FST_DEBUG("cufile: registering the file handle");
        const CUfileError_t e = g_cufile.HandleRegister(&req->cf_handle, &descr);
        FST_DEBUG("cufile: cuFileHandleRegister returned %d", (int)e.err);
        if (e.err != CU_FILE_SUCCESS) {
            set_error("gds: cuFileHandleRegister(%s) failed with cuFile error %d", path, (int)e.err);
            close(fd);
            return FST_EGDS;
        }
        req->cufile = true;
    }
    (direct ? g_counters.direct_io_requests : g_counters.buffered_io_requests).fetch_add(1);

    const uint64_t end = file_off + nbytes;
    uint64_t count = 0;
    for (uint64_t w = align_down(file_off, IO_ALIGN); w < end; w += cfg_.slot_bytes) {
        Task t;
        t.req = req;
        t.win_off = w;
        t.win_len = std::min<uint64_t>(cfg_.slot_bytes, align_up(end, IO_ALIGN) - w);
        t.valid_off = std::max(w, file_off);
        t.valid_len = std::min(end, w + t.win_len) - t.valid_off;
        t.dst = dst + dst_off + (t.valid_off - file_off);
        queue_.push_back(std::move(t));
        ++count;
    }
    req->remaining = count;
    requests_[req->id] = req;
    *out_id = req->id;
    if (count == 0) {
        if (req->cf_handle) g_cufile.HandleDeregister(req->cf_handle);
        req->cf_handle = nullptr;
        close(req->fd);
        req->fd = -1;
    }
    lock.unlock();
    work_cv_.notify_all();
    return FST_OK;
}

ssize_t Reader::do_pread(int fd, void *buf, size_t len, off_t off) {
    // the injector is for tests: the hot loop only looks at one relaxed flag unless it is armed
    if (fault_armed_.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(mu_);
        if (fault_nth_ > 0 && ++reads_seen_ == fault_nth_) {
            fault_nth_ = 0;
            fault_armed_.store(false, std::memory_order_release);
            if (fault_short_ >= 0) {
                len = (size_t)std::min<int64_t>((int64_t)len, fault_short_);
                if (len == 0) return 0;
                const ssize_t r = pread(fd, buf, len, off);
                return r;  // the caller sees a short count and must treat it as end of data
            }
            errno = fault_err_;
            return -1;
        }
    }
    return pread(fd, buf, len, off);
}

void Reader::finish(const Task &t, int status, const std::string &err, uint64_t bytes) {
    std::lock_guard<std::mutex> lock(mu_);
    Request &r = *t.req;
    if (status != FST_OK && r.status.load(std::memory_order_relaxed) == FST_OK) {
        r.status.store(status, std::memory_order_relaxed);
        r.error = err;
    }
    r.bytes_done += bytes;
    if (--r.remaining == 0) {
        if (r.cf_handle) g_cufile.HandleDeregister(r.cf_handle);
        r.cf_handle = nullptr;
        if (r.fd >= 0) close(r.fd);
        r.fd = -1;
        done_cv_.notify_all();
    }
}

void Reader::run_task(const Task &t, Slot &slot, int worker_index) {
    Request &r = *t.req;
    const bool to_device = cfg_.device >= 0;
    char msg[256];
    if (r.status.load(std::memory_order_relaxed) != FST_OK) {  // already failed: drain without I/O
        finish(t, FST_OK, "", 0);
        return;
    }
    if (r.cufile) {
        run_cufile_task(t, slot, worker_index);
        return;
    }
    const uint64_t t0 = now_ns();
    unsigned char *buf = slot.host;
    uint64_t want_off = t.win_off, want_len = t.win_len;
    bool in_place = false;
    if (!to_device && !r.direct) {  // host destination through the page cache: no bounce
        buf = (unsigned char *)(uintptr_t)t.dst;
        want_off = t.valid_off;
        want_len = t.valid_len;
        in_place = true;
    }
    if (!in_place && slot.host == nullptr) {
        if (ensure_worker_ring(worker_index) != FST_OK) {
            finish(t, FST_ENOMEM, "ring allocation failed", 0);
            return;
        }
        buf = slot.host;
    }
    if (slot.pending) {
        cudaEventSynchronize(slot.done);
        slot.pending = false;
    }
    uint64_t got = 0;
    const uint64_t need = t.valid_off + t.valid_len - want_off;  // bytes that must arrive
    while (got < need) {
        const ssize_t c = do_pread(r.fd, buf + got, want_len - got, (off_t)(want_off + got));
        if (c < 0) {
            if (errno == EINTR) continue;
            std::snprintf(msg, sizeof(msg), "pread(offset=%llu, length=%llu) failed: %s",
                          (unsigned long long)(want_off + got),
                          (unsigned long long)(want_len - got), std::strerror(errno));
            finish(t, FST_EIO, msg, 0);
            return;
        }
        if (c == 0) break;
        got += (uint64_t)c;
        if (r.direct && (got % IO_ALIGN) != 0) break;  // O_DIRECT: a ragged count means EOF
    }
    g_counters.read_ns.fetch_add(now_ns() - t0, std::memory_order_relaxed);
    g_counters.bytes_read.fetch_add(got, std::memory_order_relaxed);
    if (got < need) {
        std::snprintf(msg, sizeof(msg), "short read: wanted %llu bytes at offset %llu, got %llu",
                      (unsigned long long)need, (unsigned long long)want_off,
                      (unsigned long long)got);
        finish(t, FST_EIO, msg, 0);
        return;
    }
    if (in_place) {
        finish(t, FST_OK, "", t.valid_len);
        return;
    }
    unsigned char *src = slot.host + (t.valid_off - t.win_off);
    if (!to_device) {
        std::memcpy((void *)(uintptr_t)t.dst, src, t.valid_len);
        finish(t, FST_OK, "", t.valid_len);
        return;
    }
    cudaStream_t st = streams_[worker_index % streams_.size()];
    cudaError_t e;
    if (cfg_.plain_dma_only || (((uintptr_t)src ^ (uintptr_t)t.dst) & 15u) == 0) {
        e = cudaMemcpyAsync((void *)(uintptr_t)t.dst, src, t.valid_len, cudaMemcpyHostToDevice, st);
    } else {
        if (slot.stage == nullptr) {
            const int rc = ensure_stage_ring();
            if (rc != FST_OK) {
                finish(t, rc, "device staging ring allocation failed", 0);
                return;
            }
        }
        // 16-byte envelope of the valid bytes inside the slot (slot start is page aligned)
        const uint64_t first = t.valid_off - t.win_off;
        const uint64_t a = align_down(first, 16);
        const uint64_t b = std::min<uint64_t>(align_up(first + t.valid_len, 16), cfg_.slot_bytes);
        e = cudaMemcpyAsync(slot.stage + a, slot.host + a, b - a, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess)
            e = (cudaError_t)launch_realign((void *)(uintptr_t)t.dst, slot.stage + first,
                                            t.valid_len, (void *)st);
    }
    if (e == cudaSuccess) e = cudaEventRecord(slot.done, st);
    if (e != cudaSuccess) {
        std::snprintf(msg, sizeof(msg), "host-to-device copy failed: %s", cudaGetErrorString(e));
        finish(t, FST_ECUDA, msg, 0);
        return;
    }
    slot.pending = true;
    g_counters.bytes_h2d.fetch_add(t.valid_len, std::memory_order_relaxed);
    finish(t, FST_OK, "", t.valid_len);
}

// cuFile variant of a window: cuFileRead lands the 4096-aligned file window in the slot's device
// twin (DMA from storage where GPUDirect Storage is active, cuFile's own bounce otherwise), then
// the realign kernel moves the wanted bytes to their place (a plain vector copy when source and
// destination are congruent modulo 16).
void Reader::run_cufile_task(const Task &t, Slot &slot, int worker_index) {
    Request &r = *t.req;
    char msg[256];
    if (slot.pending) {
        cudaEventSynchronize(slot.done);
        slot.pending = false;
    }
    const uint64_t t0 = now_ns();
    const uint64_t need = t.valid_off + t.valid_len - t.win_off;
    const off_t ring_off = (off_t)(slot.stage - stage_ring_);
    uint64_t got = 0;
    while (got < need) {
        FST_DEBUG("cufile: cuFileRead(offset=%llu, size=%llu)", (unsigned long long)(t.win_off + got),
                  (unsigned long long)(t.win_len - got));
        const ssize_t c = g_cufile.Read(r.cf_handle, stage_ring_, t.win_len - got,
                                        (off_t)(t.win_off + got), ring_off + (off_t)got);
        FST_DEBUG("cufile: cuFileRead returned %zd", c);
        if (c < 0) {
            std::snprintf(msg, sizeof(msg), "gds: cuFileRead(offset=%llu) failed: %zd (errno %d)",
                          (unsigned long long)(t.win_off + got), c, errno);
            finish(t, FST_EGDS, msg, 0);
            return;
        }
        if (c == 0) break;
        got += (uint64_t)c;
    }
    g_counters.read_ns.fetch_add(now_ns() - t0, std::memory_order_relaxed);
    g_counters.bytes_read.fetch_add(got, std::memory_order_relaxed);
    if (got < need) {
        std::snprintf(msg, sizeof(msg), "gds: short cuFileRead: wanted %llu bytes at offset %llu, got %llu",
                      (unsigned long long)need, (unsigned long long)t.win_off, (unsigned long long)got);
        finish(t, FST_EIO, msg, 0);
        return;
    }
    cudaStream_t st = streams_[worker_index % streams_.size()];
    cudaError_t e = (cudaError_t)launch_realign((void *)(uintptr_t)t.dst,
                                                slot.stage + (t.valid_off - t.win_off), t.valid_len,
                                                (void *)st);
    if (e == cudaSuccess) e = cudaEventRecord(slot.done, st);
    if (e != cudaSuccess) {
        std::snprintf(msg, sizeof(msg), "gds: staging to destination copy failed: %s", cudaGetErrorString(e));
        finish(t, FST_ECUDA, msg, 0);
        return;
    }
    slot.pending = true;
    finish(t, FST_OK, "", t.valid_len);
}

void Reader::worker(int index) {
    if (cfg_.numa_node >= 0) fst_pin_numa(cfg_.numa_node);
    if (cfg_.device >= 0) cudaSetDevice(cfg_.device);
    int cursor = 0;
    for (;;) {
        Task t;
        {
            std::unique_lock<std::mutex> lock(mu_);
            work_cv_.wait(lock, [&] { return stopping_ || !queue_.empty(); });
            if (queue_.empty()) return;  // stopping and drained
            t = std::move(queue_.front());
            queue_.pop_front();
        }
        Slot &slot = slots_[(size_t)index * cfg_.slots_per_thread + cursor];
        cursor = (cursor + 1) % cfg_.slots_per_thread;
        run_task(t, slot, index);
    }
}

// The request stays registered until its copies have been drained: a wait that runs out of time
// (in either phase) can be repeated with the same id, and the request's own status and error text
// are still there when it finally completes.
int Reader::wait(int64_t id, int64_t timeout_ms, uint64_t *bytes_done) {
    std::shared_ptr<Request> req;
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    {
        std::unique_lock<std::mutex> lock(mu_);
        auto it = requests_.find(id);
        if (it == requests_.end()) {
            set_error("reader: unknown request id %lld", (long long)id);
            return FST_EINVAL;
        }
        req = it->second;
        auto ready = [&] { return req->remaining == 0; };
        if (timeout_ms < 0) {
            done_cv_.wait(lock, ready);
        } else if (!done_cv_.wait_until(lock, deadline, ready)) {
            set_error("reader: request %lld still has %llu windows to read after %lld ms",
                      (long long)id, (unsigned long long)req->remaining, (long long)timeout_ms);
            return FST_ETIMEOUT;
        }
    }
    if (bytes_done) *bytes_done = req->bytes_done;
    int rc = FST_OK;
    if (cfg_.device >= 0) {
        // every window was enqueued; drain the copy streams (bounded when a timeout was given)
        for (auto &s : streams_) {
            cudaError_t e;
            if (timeout_ms < 0) {
                e = cudaStreamSynchronize(s);
            } else {
                while ((e = cudaStreamQuery(s)) == cudaErrorNotReady) {
                    if (std::chrono::steady_clock::now() > deadline) {
                        set_error("reader: copies of request %lld not complete after %lld ms",
                                  (long long)id, (long long)timeout_ms);
                        return FST_ETIMEOUT;  // still registered: the caller may wait again
                    }
                    std::this_thread::sleep_for(std::chrono::microseconds(50));
                }
            }
            if (e != cudaSuccess) {
                set_error("reader: copy stream failed: %s", cudaGetErrorString(e));
                rc = FST_ECUDA;
                break;
            }
        }
    }
    {
        std::lock_guard<std::mutex> lock(mu_);
        requests_.erase(id);
    }
    if (rc != FST_OK) return rc;
    if (req->status != FST_OK) {
        set_error("reader: request %lld failed: %s", (long long)id, req->error.c_str());
        return req->status;
    }
    return FST_OK;
}

std::mutex g_registry_mutex;
std::unordered_set<Reader *> g_registry;

Reader *lookup(uint64_t handle) {
    std::lock_guard<std::mutex> lock(g_registry_mutex);
    Reader *r = (Reader *)(uintptr_t)handle;
    return g_registry.count(r) ? r : nullptr;
}

}  // namespace
}  // namespace fst

using namespace fst;

extern "C" int fst_reader_create(const fst_reader_config_t *cfg, uint64_t *reader) {
    clear_error();
    if (cfg == nullptr || reader == nullptr) {
        set_error("fst_reader_create: null argument");
        return FST_EINVAL;
    }
    fst_reader_config_t c = *cfg;
    if (c.threads < 1 || c.threads > 1024 || c.slots_per_thread < 1 || c.slots_per_thread > 64 ||
        c.slot_bytes == 0 || c.io_mode < FST_IO_AUTO || c.io_mode > FST_IO_CUFILE) {
        set_error("fst_reader_create: bad configuration (threads=%d, slots_per_thread=%d, "
                  "slot_bytes=%llu, io_mode=%d)", c.threads, c.slots_per_thread,
                  (unsigned long long)c.slot_bytes, c.io_mode);
        return FST_EINVAL;
    }
    c.slot_bytes = align_up(c.slot_bytes, IO_ALIGN);
    if (c.copy_streams < 1) c.copy_streams = 1;
    if (c.device >= 0) {
        if (!cuda_usable()) {
            set_error("fst_reader_create: device %d requested but there is no CUDA device",
                      c.device);
            return FST_ENOCUDA;
        }
        if (c.device >= fst_cuda_device_count()) {
            set_error("fst_reader_create: device %d does not exist", c.device);
            return FST_EINVAL;
        }
    }
    Reader *r = new Reader(c);
    {
        std::lock_guard<std::mutex> lock(g_registry_mutex);
        g_registry.insert(r);
    }
    *reader = (uint64_t)(uintptr_t)r;
    return FST_OK;
}

extern "C" int fst_reader_submit(uint64_t reader, const char *path, uint64_t file_offset,
                                 uint64_t nbytes, uint64_t dst, uint64_t dst_len,
                                 uint64_t dst_offset, int64_t *request) {
    clear_error();
    Reader *r = lookup(reader);
    if (r == nullptr || path == nullptr || request == nullptr || (dst == 0 && nbytes)) {
        set_error("fst_reader_submit: bad handle or null argument");
        return FST_EINVAL;
    }
    return r->submit(path, file_offset, nbytes, dst, dst_len, dst_offset, request);
}

extern "C" int fst_reader_wait(uint64_t reader, int64_t request, int64_t timeout_ms,
                               uint64_t *bytes_done) {
    clear_error();
    Reader *r = lookup(reader);
    if (r == nullptr) {
        set_error("fst_reader_wait: bad handle");
        return FST_EINVAL;
    }
    return r->wait(request, timeout_ms, bytes_done);
}

extern "C" int fst_reader_order_after(uint64_t reader, uint64_t stream) {
    clear_error();
    Reader *r = lookup(reader);
    if (r == nullptr) {
        set_error("fst_reader_order_after: bad handle");
        return FST_EINVAL;
    }
    return r->order_after(stream);
}

extern "C" int fst_reader_destroy(uint64_t reader) {
    clear_error();
    Reader *r = lookup(reader);
    if (r == nullptr) {
        set_error("fst_reader_destroy: bad handle");
        return FST_EINVAL;
    }
    {
        std::lock_guard<std::mutex> lock(g_registry_mutex);
        g_registry.erase(r);
    }
    delete r;
    return FST_OK;
}

extern "C" int fst_reader_inject_fault(uint64_t reader, int64_t nth, int err, int64_t short_bytes) {
    clear_error();
    Reader *r = lookup(reader);
    if (r == nullptr) {
        set_error("fst_reader_inject_fault: bad handle");
        return FST_EINVAL;
    }
    r->inject(nth, err, short_bytes);
    return FST_OK;
}

extern "C" int fst_cufile_available(void) {
    std::lock_guard<std::mutex> lock(g_cufile_mutex);
    return load_cufile_locked() ? 1 : 0;
}

extern "C" int fst_gds_supported(int device) {
    (void)device;
    // GPUDirect Storage proper needs the nvidia-fs kernel module; without it cuFile can only run
    // in its compatibility mode (POSIX reads + copies inside the library)
    return access("/proc/driver/nvidia-fs/stats", F_OK) == 0 ? 1 : 0;
}
