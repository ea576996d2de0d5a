// Host-only exercise of libfst_b200's concurrent parts, meant to be built and run under
// ThreadSanitizer or AddressSanitizer together with a sanitizer build of the library:
// several readers, each with its own worker pool, used from several caller threads at once
// (host destinations, buffered and direct I/O, odd offsets), injected read errors, a truncated
// file, timeouts, and the multi-threaded host gather.  No CUDA device is needed or touched.
// Exit code 0 and no sanitizer report = pass.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "fst_b200.h"

static std::atomic<int> g_failures{0};
#define EXPECT(cond)                                                                \
    do {                                                                            \
        if (!(cond)) {                                                              \
            std::fprintf(stderr, "%s:%d: expectation failed: %s (last error: %s)\n", \
                         __FILE__, __LINE__, #cond, fst_last_error());              \
            g_failures.fetch_add(1);                                                \
        }                                                                           \
    } while (0)

static std::vector<unsigned char> pattern(size_t n, unsigned seed) {
    std::vector<unsigned char> v(n);
    unsigned x = seed * 2654435761u + 12345u;
    for (size_t i = 0; i < n; ++i) {
        x = x * 1664525u + 1013904223u;
        v[i] = (unsigned char)(x >> 24);
    }
    return v;
}

static void write_file(const std::string &path, const std::vector<unsigned char> &data) {
    FILE *f = std::fopen(path.c_str(), "wb");
    if (!f || std::fwrite(data.data(), 1, data.size(), f) != data.size()) {
        std::fprintf(stderr, "cannot write %s\n", path.c_str());
        std::exit(2);
    }
    std::fclose(f);
}

static uint64_t make_reader(int threads, int io_mode, uint64_t slot_bytes) {
    fst_reader_config_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.device = -1;
    cfg.threads = threads;
    cfg.slots_per_thread = 2;
    cfg.io_mode = io_mode;
    cfg.slot_bytes = slot_bytes;
    cfg.copy_streams = 1;
    cfg.numa_node = -1;
    uint64_t h = 0;
    EXPECT(fst_reader_create(&cfg, &h) == FST_OK);
    return h;
}

// One caller thread: its own reader, many overlapping requests over the shared file.
static void caller(const std::string &path, const std::vector<unsigned char> &want, int id) {
    const int modes[3] = {FST_IO_BUFFERED, FST_IO_DIRECT, FST_IO_AUTO};
    const uint64_t reader = make_reader(2 + id % 3, modes[id % 3], (uint64_t)(16 + 48 * (id % 2)) << 10);
    std::vector<unsigned char> dst(want.size() + 64, 0xA5);
    struct Req { int64_t id; uint64_t off, len, dst_off; };
    std::vector<Req> reqs;
    uint64_t off = (uint64_t)(id * 37 + 1);
    while (off < want.size()) {
        uint64_t len = 1000 + (uint64_t)((off * 7919) % 300000);
        if (off + len > want.size()) len = want.size() - off;
        Req r{0, off, len, off + 13};
        EXPECT(fst_reader_submit(reader, path.c_str(), r.off, r.len, (uint64_t)dst.data(), dst.size(),
                                 r.dst_off, &r.id) == FST_OK);
        reqs.push_back(r);
        off += len + (uint64_t)(id + 1) * 4099;   // leave gaps: they must keep their canary
    }
    for (const Req &r : reqs) {
        uint64_t done = 0;
        EXPECT(fst_reader_wait(reader, r.id, 60000, &done) == FST_OK);
        EXPECT(done == r.len);
        EXPECT(std::memcmp(dst.data() + r.dst_off, want.data() + r.off, r.len) == 0);
    }
    // a destination range that does not fit is refused, and nothing is queued
    int64_t bad = 0;
    EXPECT(fst_reader_submit(reader, path.c_str(), 0, 4096, (uint64_t)dst.data(), 1000, 0, &bad) == FST_ERANGE);
    EXPECT(fst_reader_destroy(reader) == FST_OK);
}

static void failing_reads(const std::string &path, size_t size) {
    const uint64_t reader = make_reader(4, FST_IO_BUFFERED, 64 << 10);
    std::vector<unsigned char> dst(size);
    // the third pread fails with EIO: the request reports it after all windows were drained
    EXPECT(fst_reader_inject_fault(reader, 3, 5 /* EIO */, -1) == FST_OK);
    int64_t id = 0;
    uint64_t done = 0;
    EXPECT(fst_reader_submit(reader, path.c_str(), 0, size, (uint64_t)dst.data(), dst.size(), 0, &id) == FST_OK);
    EXPECT(fst_reader_wait(reader, id, 60000, &done) == FST_EIO);
    // the reader is usable afterwards
    EXPECT(fst_reader_inject_fault(reader, 0, 0, -1) == FST_OK);
    EXPECT(fst_reader_submit(reader, path.c_str(), 0, size, (uint64_t)dst.data(), dst.size(), 0, &id) == FST_OK);
    EXPECT(fst_reader_wait(reader, id, 60000, &done) == FST_OK && done == size);
    // a short pread is resumed, not reported
    EXPECT(fst_reader_inject_fault(reader, 2, 0, 100) == FST_OK);
    EXPECT(fst_reader_submit(reader, path.c_str(), 0, size, (uint64_t)dst.data(), dst.size(), 0, &id) == FST_OK);
    EXPECT(fst_reader_wait(reader, id, 60000, &done) == FST_OK && done == size);
    // a range that extends past the end of the file is refused when it is submitted
    EXPECT(fst_reader_submit(reader, path.c_str(), size - 1000, 5000, (uint64_t)dst.data(), dst.size(), 0, &id) < 0);
    // a missing file fails at submit or at wait, never hangs
    const int rc = fst_reader_submit(reader, "/nonexistent/fst_b200_file", 0, 4096, (uint64_t)dst.data(), dst.size(), 0, &id);
    if (rc == FST_OK) EXPECT(fst_reader_wait(reader, id, 60000, &done) != FST_OK);
    // an unknown request id
    EXPECT(fst_reader_wait(reader, 987654, 10, &done) == FST_EINVAL);
    EXPECT(fst_reader_destroy(reader) == FST_OK);
}

// A wait that runs out of time leaves the request registered: polling with a zero timeout until
// the request completes must end with FST_OK and the right bytes, and only then is the id
// forgotten.  Ordering a host reader behind a stream is accepted and does nothing.
static void polled_wait(const std::string &path, const std::vector<unsigned char> &want) {
    const uint64_t reader = make_reader(1, FST_IO_DIRECT, 4096);
    std::vector<unsigned char> dst(want.size());
    EXPECT(fst_reader_order_after(reader, 0) == FST_OK);
    int64_t id = 0;
    uint64_t done = 0;
    EXPECT(fst_reader_submit(reader, path.c_str(), 0, want.size(), (uint64_t)dst.data(), dst.size(), 0, &id) == FST_OK);
    int rc = FST_ETIMEOUT;
    long polls = 0;
    while (rc == FST_ETIMEOUT && polls < 50000000) {
        rc = fst_reader_wait(reader, id, 0, &done);
        ++polls;
    }
    EXPECT(rc == FST_OK && done == want.size());
    EXPECT(std::memcmp(dst.data(), want.data(), want.size()) == 0);
    EXPECT(fst_reader_wait(reader, id, 0, &done) == FST_EINVAL);
    EXPECT(fst_reader_destroy(reader) == FST_OK);
}

static void host_gather(int threads) {
    const uint64_t rows = 777, width = 3001, parts = 7;
    const std::vector<unsigned char> src = pattern(rows * width, 99);
    std::vector<unsigned char> dst(rows * width + 32, 0xA5);
    // split every row into `parts` uneven segments and pack segment k of all rows together
    std::vector<fst_copy2d_t> ops;
    uint64_t col = 0, out = 5;
    std::vector<uint64_t> seg_out;
    for (uint64_t k = 0; k < parts; ++k) {
        const uint64_t w = k + 1 < parts ? width / parts + k : width - col;
        ops.push_back(fst_copy2d_t{(uint64_t)src.data() + col, (uint64_t)dst.data() + out, rows, w, width, w});
        seg_out.push_back(out);
        col += w;
        out += rows * w;
    }
    EXPECT(fst_gather_host(ops.data(), ops.size(), threads) == FST_OK);
    col = 0;
    for (uint64_t k = 0; k < parts; ++k) {
        const uint64_t w = ops[k].row_bytes;
        for (uint64_t r = 0; r < rows; r += 97)
            EXPECT(std::memcmp(dst.data() + seg_out[k] + r * w, src.data() + r * width + col, w) == 0);
        col += w;
    }
    EXPECT(dst[4] == 0xA5 && dst[out] == 0xA5);
}

int main(int argc, char **argv) {
    const std::string dir = argc > 1 ? argv[1] : "/tmp";
    const std::string path = dir + "/fst_b200_host_stress.bin";
    const std::vector<unsigned char> data = pattern((3u << 20) + 12345u, 7);
    write_file(path, data);

    std::vector<std::thread> callers;
    for (int i = 0; i < 6; ++i) callers.emplace_back(caller, std::cref(path), std::cref(data), i);
    std::thread gather_a(host_gather, 1), gather_b(host_gather, 5);
    std::thread failing(failing_reads, std::cref(path), data.size());
    std::thread polling(polled_wait, std::cref(path), std::cref(data));
    for (auto &t : callers) t.join();
    polling.join();
    gather_a.join();
    gather_b.join();
    failing.join();

    fst_metrics_t m;
    EXPECT(fst_get_metrics(&m) == FST_OK);
    EXPECT(m.bounce_buffer_bytes == 0);     // every reader destroyed: no ring left
    EXPECT(m.bytes_read > data.size());
    std::remove(path.c_str());
    if (g_failures.load() != 0) {
        std::fprintf(stderr, "%d expectation(s) failed\n", g_failures.load());
        return 1;
    }
    std::puts("host stress ok");
    return 0;
}
