// Peer arenas of libfst_b200.so: device buffers that other processes on the same machine can
// map (CUDA IPC) so that the gather kernel of a file's owner stores each shard straight into
// the HBM of the rank that will use it, over NVLink, with ordinary 16-byte stores.
//
// An arena is a plain cudaMalloc allocation (IPC handles cannot name memory that comes from a
// framework's sub-allocator).  The exporter keeps it until every importer has closed its
// mapping; the loader enforces that order with a barrier.
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>
#include <unordered_map>

#include "fst_internal.h"

namespace fst {
namespace {

struct Arena {
    void *base = nullptr;
    uint64_t nbytes = 0;
    int device = 0;
};
std::mutex g_arena_mutex;
std::unordered_map<uint64_t, Arena> g_arenas;        // handle (= base address) -> arena
std::unordered_map<uint64_t, int> g_peer_mappings;   // mapped peer address -> device it was opened on

}  // namespace
}  // namespace fst

using namespace fst;

extern "C" int fst_arena_create(uint64_t nbytes, uint64_t *arena) {
    clear_error();
    if (arena == nullptr) {
        set_error("fst_arena_create: null argument");
        return FST_EINVAL;
    }
    if (!cuda_usable()) {
        set_error("fst_arena_create: no CUDA device");
        return FST_ENOCUDA;
    }
    Arena a;
    cudaGetDevice(&a.device);
    a.nbytes = nbytes ? nbytes : 256;
    const cudaError_t e = cudaMalloc(&a.base, a.nbytes);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        set_error("fst_arena_create: cudaMalloc(%llu) failed: %s", (unsigned long long)a.nbytes,
                  cudaGetErrorString(e));
        return FST_ENOMEM;
    }
    std::lock_guard<std::mutex> lock(g_arena_mutex);
    g_arenas[(uint64_t)(uintptr_t)a.base] = a;
    *arena = (uint64_t)(uintptr_t)a.base;
    return FST_OK;
}

extern "C" int fst_arena_export(uint64_t arena, void *handle, uint64_t handle_bytes) {
    clear_error();
    if (handle == nullptr || handle_bytes < sizeof(cudaIpcMemHandle_t)) {
        set_error("fst_arena_export: handle buffer must hold %zu bytes", sizeof(cudaIpcMemHandle_t));
        return FST_EINVAL;
    }
    {
        std::lock_guard<std::mutex> lock(g_arena_mutex);
        if (!g_arenas.count(arena)) {
            set_error("fst_arena_export: unknown arena");
            return FST_EINVAL;
        }
    }
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, (void *)(uintptr_t)arena);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        set_error("fst_arena_export: cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
        return FST_ECUDA;
    }
    std::memset(handle, 0, handle_bytes);
    std::memcpy(handle, &h, sizeof(h));
    return FST_OK;
}

extern "C" int fst_arena_open_peer(const void *handle, uint64_t handle_bytes, uint64_t *peer_addr) {
    clear_error();
    if (handle == nullptr || peer_addr == nullptr || handle_bytes < sizeof(cudaIpcMemHandle_t)) {
        set_error("fst_arena_open_peer: bad argument");
        return FST_EINVAL;
    }
    if (!cuda_usable()) {
        set_error("fst_arena_open_peer: no CUDA device");
        return FST_ENOCUDA;
    }
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    void *p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess || p == nullptr) {
        (void)cudaGetLastError();
        set_error("fst_arena_open_peer: cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
        return FST_ECUDA;
    }
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(g_arena_mutex);
    g_peer_mappings[(uint64_t)(uintptr_t)p] = dev;
    *peer_addr = (uint64_t)(uintptr_t)p;
    return FST_OK;
}

extern "C" int fst_arena_close_peer(uint64_t peer_addr) {
    clear_error();
    {
        std::lock_guard<std::mutex> lock(g_arena_mutex);
        if (!g_peer_mappings.erase(peer_addr)) {
            set_error("fst_arena_close_peer: address was not opened with fst_arena_open_peer");
            return FST_EINVAL;
        }
    }
    const cudaError_t e = cudaIpcCloseMemHandle((void *)(uintptr_t)peer_addr);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        set_error("fst_arena_close_peer: cudaIpcCloseMemHandle failed: %s", cudaGetErrorString(e));
        return FST_ECUDA;
    }
    return FST_OK;
}

extern "C" int fst_arena_destroy(uint64_t arena) {
    clear_error();
    {
        std::lock_guard<std::mutex> lock(g_arena_mutex);
        if (!g_arenas.erase(arena)) {
            set_error("fst_arena_destroy: unknown arena");
            return FST_EINVAL;
        }
    }
    const cudaError_t e = cudaFree((void *)(uintptr_t)arena);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        set_error("fst_arena_destroy: cudaFree failed: %s", cudaGetErrorString(e));
        return FST_ECUDA;
    }
    return FST_OK;
}
