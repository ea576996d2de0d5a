// Host-side utilities of libfst_b200.so: error text, counters, topology, NUMA binding, host
// allocation and the host-memory variant of the gather (the loader's CPU mode).
#include <cuda_runtime.h>
#include <sched.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <cerrno>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <fstream>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "fst_internal.h"

namespace fst {

std::atomic<int> g_debug{0};
Counters g_counters;

namespace {
thread_local char t_error[512] = "";
}

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    std::vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
    FST_DEBUG("error: %s", t_error);
}

void clear_error() { t_error[0] = '\0'; }

bool cuda_usable() {
    static int state = -1;  // -1 unknown, 0 no, 1 yes
    static std::mutex m;
    std::lock_guard<std::mutex> lock(m);
    if (state < 0) {
        int n = 0;
        const cudaError_t e = cudaGetDeviceCount(&n);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();  // do not leave a sticky "no device" error behind
            n = 0;
        }
        state = n > 0 ? 1 : 0;
    }
    return state == 1;
}

namespace {

// "0-3,8-11" -> cpu list
std::vector<int> parse_cpulist(const std::string &s) {
    std::vector<int> cpus;
    size_t i = 0;
    while (i < s.size()) {
        char *end = nullptr;
        const long a = std::strtol(s.c_str() + i, &end, 10);
        if (end == s.c_str() + i) break;
        long b = a;
        i = (size_t)(end - s.c_str());
        if (i < s.size() && s[i] == '-') {
            b = std::strtol(s.c_str() + i + 1, &end, 10);
            i = (size_t)(end - s.c_str());
        }
        for (long c = a; c <= b; ++c) cpus.push_back((int)c);
        if (i < s.size() && s[i] == ',') ++i;
        else break;
    }
    return cpus;
}

}  // namespace
}  // namespace fst

using namespace fst;

extern "C" int fst_abi_version(void) { return FST_B200_ABI_VERSION; }

extern "C" const char *fst_last_error(void) { return t_error; }

extern "C" int fst_cuda_device_count(void) {
    if (!cuda_usable()) return 0;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
    return n;
}

extern "C" void fst_set_debug(int on) { g_debug.store(on ? 1 : 0); }

extern "C" uint64_t fst_device_alloc(uint64_t nbytes) {
    clear_error();
    if (!cuda_usable()) {
        set_error("fst_device_alloc: no CUDA device");
        return 0;
    }
    void *p = nullptr;
    const cudaError_t e = cudaMalloc(&p, nbytes);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        set_error("fst_device_alloc: cudaMalloc(%llu) failed: %s", (unsigned long long)nbytes,
                  cudaGetErrorString(e));
        return 0;
    }
    return (uint64_t)(uintptr_t)p;
}

extern "C" void fst_device_free(uint64_t addr) {
    if (addr != 0 && cuda_usable()) cudaFree((void *)(uintptr_t)addr);
}

extern "C" int fst_memcpy_h2d_async(uint64_t dst, uint64_t src, uint64_t nbytes) {
    clear_error();
    if (!cuda_usable()) {
        set_error("fst_memcpy_h2d_async: no CUDA device");
        return FST_ENOCUDA;
    }
    const cudaError_t e = cudaMemcpyAsync((void *)(uintptr_t)dst, (const void *)(uintptr_t)src,
                                          nbytes, cudaMemcpyHostToDevice, nullptr);
    if (e != cudaSuccess) (void)cudaGetLastError();
    return (int)e;
}

extern "C" int fst_device_pci_bus(int device, char *out, int n) {
    clear_error();
    if (out == nullptr || n < 16) {
        set_error("fst_device_pci_bus: output buffer too small");
        return FST_EINVAL;
    }
    out[0] = '\0';
    if (!cuda_usable()) {
        set_error("fst_device_pci_bus: no CUDA device");
        return FST_ENOCUDA;
    }
    const cudaError_t e = cudaDeviceGetPCIBusId(out, n, device);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        set_error("fst_device_pci_bus: cudaDeviceGetPCIBusId(%d): %s", device,
                  cudaGetErrorString(e));
        return FST_ECUDA;
    }
    return FST_OK;
}

extern "C" int fst_device_numa_node(int device) {
    char bus[64];
    if (fst_device_pci_bus(device, bus, sizeof(bus)) != FST_OK) return -1;
    std::string id(bus);
    for (auto &c : id) c = (char)std::tolower((unsigned char)c);
    std::ifstream f("/sys/bus/pci/devices/" + id + "/numa_node");
    int node = -1;
    if (f && (f >> node)) return node;
    return -1;
}

extern "C" int fst_pin_numa(int node) {
    clear_error();
    if (node < 0) return FST_OK;
    std::ifstream f("/sys/devices/system/node/node" + std::to_string(node) + "/cpulist");
    std::string line;
    if (!f || !std::getline(f, line)) {
        set_error("fst_pin_numa: node %d has no cpulist in sysfs", node);
        return FST_EINVAL;
    }
    const std::vector<int> cpus = parse_cpulist(line);
    if (cpus.empty()) {
        set_error("fst_pin_numa: node %d has no CPUs", node);
        return FST_EINVAL;
    }
    cpu_set_t set;
    CPU_ZERO(&set);
    for (int c : cpus)
        if (c >= 0 && c < CPU_SETSIZE) CPU_SET(c, &set);
    if (sched_setaffinity(0, sizeof(set), &set) != 0) {
        set_error("fst_pin_numa: sched_setaffinity: %s", std::strerror(errno));
        return FST_EINVAL;
    }
#ifdef SYS_set_mempolicy
    if (node < 1024) {
        // MPOL_PREFERRED = 1: new pages (the pinned ring among them) come from this node
        unsigned long mask[16] = {};
        mask[node / (8 * sizeof(unsigned long))] |= 1ul << (node % (8 * sizeof(unsigned long)));
        (void)syscall(SYS_set_mempolicy, 1, mask, (unsigned long)(sizeof(mask) * 8));
    }
#endif
    return FST_OK;
}

extern "C" uint64_t fst_host_alloc(uint64_t nbytes) {
    void *p = nullptr;
    if (posix_memalign(&p, 4096, nbytes ? nbytes : 1) != 0) return 0;
    return (uint64_t)(uintptr_t)p;
}

extern "C" void fst_host_free(uint64_t addr) { std::free((void *)(uintptr_t)addr); }

extern "C" int fst_read_host(uint64_t addr, uint64_t nbytes, void *out) {
    clear_error();
    if ((addr == 0 || out == nullptr) && nbytes) {
        set_error("fst_read_host: null address");
        return FST_EINVAL;
    }
    std::memcpy(out, (const void *)(uintptr_t)addr, nbytes);
    return FST_OK;
}

extern "C" int fst_io_alignment(void) { return 4096; }

extern "C" int fst_get_metrics(fst_metrics_t *out) {
    if (out == nullptr) return FST_EINVAL;
    std::memset(out, 0, sizeof(*out));
    out->bounce_buffer_bytes = g_counters.bounce_buffer_bytes.load();
    out->staging_device_bytes = g_counters.staging_device_bytes.load();
    out->bytes_read = g_counters.bytes_read.load();
    out->bytes_h2d = g_counters.bytes_h2d.load();
    out->bytes_realigned = g_counters.bytes_realigned.load();
    out->bytes_gathered = g_counters.bytes_gathered.load();
    out->kernel_launches = g_counters.kernel_launches.load();
    out->direct_io_requests = g_counters.direct_io_requests.load();
    out->buffered_io_requests = g_counters.buffered_io_requests.load();
    out->read_ns = g_counters.read_ns.load();
    return FST_OK;
}

extern "C" int fst_gather_host(const fst_copy2d_t *ops, uint64_t n_ops, int threads) {
    clear_error();
    if (n_ops == 0) return FST_OK;
    if (ops == nullptr) {
        set_error("fst_gather_host: ops is null");
        return FST_EINVAL;
    }
    uint64_t total = 0;
    for (uint64_t i = 0; i < n_ops; ++i) {
        const fst_copy2d_t &c = ops[i];
        if (c.rows == 0 || c.row_bytes == 0) continue;
        if (c.src == 0 || c.dst == 0) {
            set_error("fst_gather_host: op %llu has a null address", (unsigned long long)i);
            return FST_EINVAL;
        }
        if (c.rows > 1 && (c.src_pitch < c.row_bytes || c.dst_pitch < c.row_bytes)) {
            set_error("fst_gather_host: op %llu: pitch smaller than row_bytes",
                      (unsigned long long)i);
            return FST_EINVAL;
        }
        total += c.rows * c.row_bytes;
    }
    // rows longer than 1 MiB are cut into pieces so that one huge row (a dim-0 shard) is
    // still shared by all threads
    std::vector<fst_copy2d_t> norm;
    norm.reserve(n_ops);
    constexpr uint64_t PIECE = 1u << 20;
    for (uint64_t i = 0; i < n_ops; ++i) {
        const fst_copy2d_t &c = ops[i];
        if (c.rows == 0 || c.row_bytes == 0) continue;
        if (c.row_bytes <= PIECE) {
            norm.push_back(c);
            continue;
        }
        for (uint64_t r = 0; r < c.rows; ++r)
            for (uint64_t o = 0; o < c.row_bytes; o += PIECE) {
                fst_copy2d_t p = {c.src + r * c.src_pitch + o, c.dst + r * c.dst_pitch + o, 1,
                                  std::min<uint64_t>(PIECE, c.row_bytes - o), 0, 0};
                norm.push_back(p);
            }
    }
    ops = norm.data();
    n_ops = norm.size();
    // rows of all ops are dealt out in contiguous shares, one share per thread
    int nt = threads < 1 ? 1 : threads;
    if (total < (1u << 20)) nt = 1;
    auto run = [&](int t) {
        const uint64_t lo = total / nt * t, hi = (t == nt - 1) ? total : total / nt * (t + 1);
        uint64_t pos = 0;  // payload bytes before the current op
        for (uint64_t i = 0; i < n_ops && pos < hi; ++i) {
            const fst_copy2d_t &c = ops[i];
            const uint64_t bytes = c.rows * c.row_bytes;
            if (bytes == 0) continue;
            if (pos + bytes > lo) {
                // this thread copies the rows whose first byte falls in [lo, hi)
                uint64_t r0 = pos >= lo ? 0 : (lo - pos + c.row_bytes - 1) / c.row_bytes;
                uint64_t r1 = pos + bytes <= hi ? c.rows : (hi - pos + c.row_bytes - 1) / c.row_bytes;
                for (uint64_t r = r0; r < r1; ++r)
                    std::memcpy((void *)(uintptr_t)(c.dst + r * c.dst_pitch),
                                (const void *)(uintptr_t)(c.src + r * c.src_pitch), c.row_bytes);
            }
            pos += bytes;
        }
    };
    if (nt == 1) {
        run(0);
    } else {
        std::vector<std::thread> pool;
        for (int t = 1; t < nt; ++t) pool.emplace_back(run, t);
        run(0);
        for (auto &th : pool) th.join();
    }
    return FST_OK;
}
