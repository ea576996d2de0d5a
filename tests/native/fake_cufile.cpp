// A host-side double of the seven cuFile entry points libfst_b200.so resolves, for tests.
//
// It never touches NVIDIA's libcufile, the cuFile driver or the nvidia-fs module: a "cuFileRead"
// is a pread into host memory followed by a copy to devPtr_base + devPtr_offset that is complete
// when the call returns.  That is enough to run the reader's cuFile code path (driver reference count,
// register-once staging ring, per-request file handles, 4096-aligned windows into staging slots,
// realign kernel to the destination) on any machine with a CUDA device.  The marker symbol
// `fst_cufile_stand_in` tells the reader that this library needs no nvidia-fs.
//
// The same idea as upstream's table of fake cuFile functions (fastsafetensors/cpp/ext.cpp:126-196,
// used by tests/unit/test_fastsafetensors.py:361-376), kept outside the product library.
//
// Build: g++ -shared -fPIC fake_cufile.cpp -I$CUDA/include -L$CUDA/lib64 -lcudart -o libfake_cufile.so
#include <cuda_runtime.h>
#include <cufile.h>
#include <unistd.h>
#undef cuFileDriverClose  // the header renames it to cuFileDriverClose_v2; both names are exported

#include <atomic>
#include <cerrno>
#include <cstdint>
#include <cstdlib>
#include <mutex>
#include <set>

namespace {

struct Handle {
    int fd;
};

std::mutex g_mu;
std::set<const void *> g_registered;
std::set<Handle *> g_handles;
std::atomic<int64_t> g_driver_open{0}, g_driver_close{0}, g_buf_register{0}, g_buf_deregister{0},
    g_handle_register{0}, g_handle_deregister{0}, g_reads{0}, g_read_bytes{0},
    g_reads_into_registered{0}, g_fail_read_at{0};

CUfileError_t ok() {
    CUfileError_t e;
    e.err = CU_FILE_SUCCESS;
    e.cu_err = CUDA_SUCCESS;
    return e;
}

CUfileError_t bad(CUfileOpError code) {
    CUfileError_t e;
    e.err = code;
    e.cu_err = CUDA_SUCCESS;
    return e;
}

}  // namespace

extern "C" {

__attribute__((visibility("default"))) int fst_cufile_stand_in = 1;

__attribute__((visibility("default"))) CUfileError_t cuFileDriverOpen(void) {
    ++g_driver_open;
    return ok();
}

__attribute__((visibility("default"))) CUfileError_t cuFileDriverClose(void) {
    ++g_driver_close;
    return ok();
}

__attribute__((visibility("default"))) CUfileError_t cuFileDriverClose_v2(void) {
    return cuFileDriverClose();
}

__attribute__((visibility("default"))) CUfileError_t cuFileHandleRegister(CUfileHandle_t *fh,
                                                                          CUfileDescr_t *descr) {
    if (fh == nullptr || descr == nullptr || descr->type != CU_FILE_HANDLE_TYPE_OPAQUE_FD ||
        descr->handle.fd < 0)
        return bad(CU_FILE_INVALID_VALUE);
    Handle *h = new Handle{descr->handle.fd};
    {
        std::lock_guard<std::mutex> lock(g_mu);
        g_handles.insert(h);
    }
    *fh = (CUfileHandle_t)h;
    ++g_handle_register;
    return ok();
}

__attribute__((visibility("default"))) void cuFileHandleDeregister(CUfileHandle_t fh) {
    Handle *h = (Handle *)fh;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (!g_handles.erase(h)) return;
    }
    delete h;
    ++g_handle_deregister;
}

__attribute__((visibility("default"))) CUfileError_t cuFileBufRegister(const void *devPtr,
                                                                       size_t length, int flags) {
    (void)flags;
    if (devPtr == nullptr || length == 0) return bad(CU_FILE_INVALID_VALUE);
    std::lock_guard<std::mutex> lock(g_mu);
    g_registered.insert(devPtr);
    ++g_buf_register;
    return ok();
}

__attribute__((visibility("default"))) CUfileError_t cuFileBufDeregister(const void *devPtr) {
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_registered.erase(devPtr)) return bad(CU_FILE_INVALID_VALUE);
    ++g_buf_deregister;
    return ok();
}

__attribute__((visibility("default"))) ssize_t cuFileRead(CUfileHandle_t fh, void *devPtr_base,
                                                          size_t size, off_t file_offset,
                                                          off_t devPtr_offset) {
    Handle *h = (Handle *)fh;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (!g_handles.count(h)) return -1;
        if (g_registered.count(devPtr_base)) ++g_reads_into_registered;
    }
    const int64_t nth = ++g_reads;
    if (g_fail_read_at.load() == nth) {
        errno = EIO;
        return -1;
    }
    // page-aligned bounce: the reader opens its files with O_DIRECT for cuFile
    void *host = nullptr;
    if (posix_memalign(&host, 4096, (size + 4095) / 4096 * 4096) != 0) return -1;
    size_t got = 0;
    while (got < size) {
        const ssize_t c = pread(h->fd, (unsigned char *)host + got, size - got, file_offset + (off_t)got);
        if (c < 0) {
            if (errno == EINTR) continue;
            std::free(host);
            return -1;
        }
        if (c == 0) break;  // end of file: a short count, as cuFileRead reports it
        got += (size_t)c;
        if (got % 4096) break;  // a ragged count under O_DIRECT means end of file
    }
    // cuFileRead returns when the bytes ARE in device memory.  A plain cudaMemcpy from pageable
    // memory may return while its DMA is still in flight, so the copy goes through a stream of
    // this thread's own and waits for it.
    static thread_local cudaStream_t stream = nullptr;
    bool ok = true;
    if (got) {
        if (stream == nullptr) ok = cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) == cudaSuccess;
        ok = ok && cudaMemcpyAsync((unsigned char *)devPtr_base + devPtr_offset, host, got,
                                   cudaMemcpyHostToDevice, stream) == cudaSuccess;
        ok = ok && cudaStreamSynchronize(stream) == cudaSuccess;
    }
    std::free(host);
    if (!ok) return -1;
    g_read_bytes += (int64_t)got;
    return (ssize_t)got;
}

// Test hooks (not part of cuFile): counters, and "fail the n-th read from now on".
__attribute__((visibility("default"))) void fake_cufile_counts(int64_t out[10]) {
    std::lock_guard<std::mutex> lock(g_mu);
    out[0] = g_driver_open;
    out[1] = g_driver_close;
    out[2] = g_buf_register;
    out[3] = g_buf_deregister;
    out[4] = g_handle_register;
    out[5] = g_handle_deregister;
    out[6] = g_reads;
    out[7] = g_read_bytes;
    out[8] = g_reads_into_registered;
    out[9] = (int64_t)g_handles.size();
}

__attribute__((visibility("default"))) void fake_cufile_fail_read(int64_t nth_from_now) {
    g_fail_read_at = nth_from_now > 0 ? g_reads.load() + nth_from_now : 0;
}

}  // extern "C"
