// Internal declarations shared by the translation units of libfst_b200.so.
// Nothing here is part of the C ABI (see include/fst_b200.h for that).
#ifndef FST_INTERNAL_H
#define FST_INTERNAL_H

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "fst_b200.h"

namespace fst {

// Thread-local error text behind fst_last_error().
void set_error(const char *fmt, ...) __attribute__((format(printf, 1, 2)));
void clear_error();

extern std::atomic<int> g_debug;

// Process-wide counters behind fst_get_metrics().
struct Counters {
    std::atomic<uint64_t> bounce_buffer_bytes{0};
    std::atomic<uint64_t> staging_device_bytes{0};
    std::atomic<uint64_t> bytes_read{0};
    std::atomic<uint64_t> bytes_h2d{0};
    std::atomic<uint64_t> bytes_realigned{0};
    std::atomic<uint64_t> bytes_gathered{0};
    std::atomic<uint64_t> kernel_launches{0};
    std::atomic<uint64_t> direct_io_requests{0};
    std::atomic<uint64_t> buffered_io_requests{0};
    std::atomic<uint64_t> read_ns{0};
};
extern Counters g_counters;

// True when a CUDA driver and at least one device are usable (cached after the first call).
bool cuda_usable();

// Enqueue the realign kernel (no argument checks; callers validate).  Returns a cudaError_t.
int launch_realign(void *dst, const void *src, uint64_t nbytes, void *stream);

}  // namespace fst

#define FST_DEBUG(...)                        \
    do {                                      \
        if (fst::g_debug.load(std::memory_order_relaxed)) { \
            std::printf("[fst_b200] " __VA_ARGS__);          \
            std::printf("\n");                \
        }                                     \
    } while (0)

#endif  // FST_INTERNAL_H
