// Device kernels of libfst_b200.so (sm_100a): shard gather/pack and realign.
//
// Both are pure byte movers bound by HBM bandwidth: every payload byte is read once and
// written once (algorithmic traffic = 2 x payload).  The design rules are the ones that matter
// for such a kernel on B200: 16-byte global loads and stores that a warp issues as whole
// 512-byte rows (fully coalesced sectors on both sides), eight independent 16-byte loads in
// flight per lane before the first store, streaming cache hints (the data is touched once),
// and many short CTAs rather than a persistent grid (see grid_limit_for for the measurement).
//
// Work decomposition (gather).  An op is a strided 2-D byte copy (fst_copy2d_t).  Each row of
// an op is cut into "subs" of at most SUB_BYTES; a sub is copied by one warp.  Sub boundaries
// are placed so that, when the destination pitch allows it, every sub except the first of a
// row starts on a 16-byte destination boundary.  Subs of all ops are numbered consecutively;
// a warp finds the op of a sub by binary search over the ops' first-sub prefix.
//
// Short rows.  A row of at most SHORT_ROW_BYTES (a column split of a narrow or an 8-bit / 4-bit
// matrix) would leave most of a warp idle if it were a sub of its own.  For such ops a sub holds
// several whole rows instead: the warp is divided into groups of 1, 2, 4, 8 or 16 lanes (64
// bytes of row per lane), each group copies one row with its own head / body / tail, and a sub
// is 32 / group rows.
//
// Alignment.  A sub is copied as: up to 15 head bytes (until the destination is 16-byte
// aligned), a body of 16-byte destination vectors, up to 15 tail bytes.  If the source is
// congruent to the destination modulo 16 the body is a plain vector copy; if not, each
// destination vector is assembled from the two aligned 16-byte source words that straddle it
// with funnel shifts (a lane loads the first and gets the second from the next lane by
// shuffle).  The aligned words read may extend up to 15 bytes before or after the
// source range, but always inside a 16-byte word that holds at least one byte of the range, so
// they never touch another page.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "fst_internal.h"

namespace fst {

constexpr int SUB_BYTES = 2048;          // bytes one warp moves per sub (32 lanes x 4 x 16 B)
constexpr int VEC_PER_LANE = SUB_BYTES / (32 * 16);
constexpr int WARPS_PER_CTA = 8;
constexpr int CTA_THREADS = WARPS_PER_CTA * 32;
constexpr int SUBS_PER_WARP_STEP = 2;    // subs a warp loads before it starts storing
constexpr int SHORT_ROW_BYTES = SUB_BYTES / 2;   // rows up to this size share a sub
constexpr int LANE_BYTES = VEC_PER_LANE * 16;    // bytes of one row a lane can hold in registers

// Device-side record of one op (64 bytes).
struct GatherOp {
    uint64_t src;
    uint64_t dst;
    uint64_t src_pitch;
    uint64_t dst_pitch;
    uint64_t row_bytes;
    uint32_t subs_per_row;  // 0 marks a short-row op (a sub is several whole rows)
    uint32_t lead;          // long rows: (dst & 15) when every row has the same destination
                            // alignment, else 0; short rows: lanes that share one row
    uint64_t first_sub;     // number of subs in all earlier ops
    uint64_t rows;
};
static_assert(sizeof(GatherOp) == 64, "GatherOp must stay 64 bytes");

struct InlineOps {
    GatherOp op[FST_GATHER_INLINE_OPS];
};

__device__ __forceinline__ uint4 ld_stream(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint4 ld_keep(const uint4 *p) {
    // neighbouring lanes re-read this word in the shifted path: let it live in L1
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void st_stream(uint4 *p, const uint4 &v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w)
                 : "memory");
}

// Bytes [shift, shift+16) of the 32-byte pair (lo, hi); shift in 1..15.
__device__ __forceinline__ uint4 funnel16(const uint4 &lo, const uint4 &hi, unsigned shift) {
    const unsigned bits = (shift & 3u) * 8u;
    uint4 r;
    switch (shift >> 2) {
        case 0:
            r.x = __funnelshift_r(lo.x, lo.y, bits);
            r.y = __funnelshift_r(lo.y, lo.z, bits);
            r.z = __funnelshift_r(lo.z, lo.w, bits);
            r.w = __funnelshift_r(lo.w, hi.x, bits);
            break;
        case 1:
            r.x = __funnelshift_r(lo.y, lo.z, bits);
            r.y = __funnelshift_r(lo.z, lo.w, bits);
            r.z = __funnelshift_r(lo.w, hi.x, bits);
            r.w = __funnelshift_r(hi.x, hi.y, bits);
            break;
        case 2:
            r.x = __funnelshift_r(lo.z, lo.w, bits);
            r.y = __funnelshift_r(lo.w, hi.x, bits);
            r.z = __funnelshift_r(hi.x, hi.y, bits);
            r.w = __funnelshift_r(hi.y, hi.z, bits);
            break;
        default:
            r.x = __funnelshift_r(lo.w, hi.x, bits);
            r.y = __funnelshift_r(hi.x, hi.y, bits);
            r.z = __funnelshift_r(hi.y, hi.z, bits);
            r.w = __funnelshift_r(hi.z, hi.w, bits);
            break;
    }
    return r;
}

// One sub as seen by a warp after head/tail splitting.
struct Span {
    const unsigned char *src;  // first body byte (destination-aligned position)
    unsigned char *dst;        // 16-byte aligned
    unsigned nvec;             // body vectors (<= SUB_BYTES/16)
    unsigned shift;            // src & 15
    unsigned glane;            // this lane's index among the lanes that copy the span
    unsigned glanes;           // how many lanes copy it (32, or fewer for short rows)
};

// Copies the head and tail bytes of [dst, dst+n) <- [src, src+n) and returns the body.
__device__ __forceinline__ Span split_span(unsigned char *dst, const unsigned char *src,
                                           unsigned n, unsigned glane, unsigned glanes) {
    unsigned head = (16u - (unsigned)((uintptr_t)dst & 15u)) & 15u;
    if (head > n) head = n;
    for (unsigned b = glane; b < head; b += glanes) dst[b] = src[b];
    dst += head;
    src += head;
    n -= head;
    const unsigned nvec = n >> 4;
    const unsigned tail = n & 15u;
    for (unsigned b = glane; b < tail; b += glanes) dst[(nvec << 4) + b] = src[(nvec << 4) + b];
    Span s;
    s.src = src;
    s.dst = dst;
    s.nvec = nvec;
    s.shift = (unsigned)((uintptr_t)src & 15u);
    s.glane = glane;
    s.glanes = glanes;
    return s;
}

__device__ __forceinline__ uint4 shfl_down1(const uint4 &x, unsigned width) {
    uint4 r;
    r.x = __shfl_down_sync(0xffffffffu, x.x, 1, width);
    r.y = __shfl_down_sync(0xffffffffu, x.y, 1, width);
    r.z = __shfl_down_sync(0xffffffffu, x.z, 1, width);
    r.w = __shfl_down_sync(0xffffffffu, x.w, 1, width);
    return r;
}

__device__ __forceinline__ uint4 shfl_first(const uint4 &x, unsigned width) {
    uint4 r;
    r.x = __shfl_sync(0xffffffffu, x.x, 0, width);
    r.y = __shfl_sync(0xffffffffu, x.y, 0, width);
    r.z = __shfl_sync(0xffffffffu, x.z, 0, width);
    r.w = __shfl_sync(0xffffffffu, x.w, 0, width);
    return r;
}

// Loads the body of a span into registers.  Must be called by all 32 lanes of a warp together,
// with spans of one sub (so `glanes` is the same in every lane): the misaligned case exchanges
// words between lanes.
//
// Misaligned source: destination vector i needs the aligned source words i and i+1.  Word i+1 is
// what the next lane of the group loads as ITS word for the same j (or, for the last lane of the
// group, what the first lane loads for j+1), so every lane loads one word per vector (plus one
// more word per group) and gets the second from a shuffle, instead of loading both.
__device__ __forceinline__ void load_span(const Span &s, uint4 (&v)[VEC_PER_LANE]) {
    if (!__any_sync(0xffffffffu, s.shift != 0 && s.nvec != 0)) {   // same answer in every lane
        const uint4 *p = reinterpret_cast<const uint4 *>(s.src);
#pragma unroll
        for (int j = 0; j < VEC_PER_LANE; ++j) {
            const unsigned i = s.glane + s.glanes * j;
            if (i < s.nvec) v[j] = ld_stream(p + i);
        }
        return;
    }
    // Words to load: 0 .. nvec-1, and word nvec too when this lane's row is misaligned (it then
    // holds at least one byte of the row, see the note on alignment at the top of the file).
    const uint4 *p = reinterpret_cast<const uint4 *>(s.src - s.shift);
    const unsigned words = s.nvec == 0 ? 0u : s.nvec + (s.shift != 0 ? 1u : 0u);
    uint4 lo[VEC_PER_LANE + 1];
#pragma unroll
    for (int j = 0; j <= VEC_PER_LANE; ++j) {
        const unsigned i = s.glane + s.glanes * j;
        lo[j] = make_uint4(0u, 0u, 0u, 0u);
        if (i < words) lo[j] = ld_stream(p + i);
    }
    const bool last = s.glane + 1u == s.glanes;
#pragma unroll
    for (int j = 0; j < VEC_PER_LANE; ++j) {
        const uint4 from_next_lane = shfl_down1(lo[j], s.glanes);
        const uint4 from_first_lane = shfl_first(lo[j + 1], s.glanes);
        const uint4 hi = last ? from_first_lane : from_next_lane;
        v[j] = s.shift != 0 ? funnel16(lo[j], hi, s.shift) : lo[j];
    }
}

__device__ __forceinline__ void store_span(const Span &s, const uint4 (&v)[VEC_PER_LANE]) {
    uint4 *p = reinterpret_cast<uint4 *>(s.dst);
#pragma unroll
    for (int j = 0; j < VEC_PER_LANE; ++j) {
        const unsigned i = s.glane + s.glanes * j;
        if (i < s.nvec) st_stream(p + i, v[j]);
    }
}

// Index of the op that holds global sub g (ops sorted by first_sub, op[0].first_sub == 0).
__device__ __forceinline__ unsigned find_op(const GatherOp *ops, unsigned n_ops, uint64_t g) {
    unsigned lo = 0, hi = n_ops;  // invariant: ops[lo].first_sub <= g < ops[hi].first_sub
    while (hi - lo > 1) {
        const unsigned mid = (lo + hi) >> 1;
        if (ops[mid].first_sub <= g) lo = mid; else hi = mid;
    }
    return lo;
}

__device__ __forceinline__ Span open_sub(const GatherOp *ops, unsigned n_ops, uint64_t g,
                                         unsigned lane) {
    const GatherOp &op = ops[find_op(ops, n_ops, g)];
    const uint64_t local = g - op.first_sub;
    if (op.subs_per_row == 0) {
        // short rows: `glanes` lanes (a power of two) per row, 32 / glanes rows per sub
        const unsigned glanes = op.lead;
        const unsigned shift = (unsigned)__ffs((int)glanes) - 1u;
        const uint64_t row = (local << (5u - shift)) + (lane >> shift);
        if (row >= op.rows) {
            Span none;
            none.src = nullptr;
            none.dst = nullptr;
            none.nvec = 0;
            none.shift = 0;
            none.glane = lane & (glanes - 1u);
            none.glanes = glanes;     // the same in every lane of the warp, as load_span needs
            return none;
        }
        return split_span(reinterpret_cast<unsigned char *>(op.dst + row * op.dst_pitch),
                          reinterpret_cast<const unsigned char *>(op.src + row * op.src_pitch),
                          (unsigned)op.row_bytes, lane & (glanes - 1u), glanes);
    }
    const uint64_t row = local / op.subs_per_row;
    const unsigned k = (unsigned)(local - row * op.subs_per_row);
    // sub k of a row covers row bytes [k*SUB - lead, (k+1)*SUB - lead) clipped to the row
    uint64_t beg = (uint64_t)k * SUB_BYTES;
    beg = beg > op.lead ? beg - op.lead : 0;
    uint64_t end = (uint64_t)(k + 1) * SUB_BYTES - op.lead;
    if (end > op.row_bytes) end = op.row_bytes;
    unsigned char *d = reinterpret_cast<unsigned char *>(op.dst + row * op.dst_pitch + beg);
    const unsigned char *s =
        reinterpret_cast<const unsigned char *>(op.src + row * op.src_pitch + beg);
    return split_span(d, s, (unsigned)(end - beg), lane, 32u);
}

template <bool INLINE>
__global__ void __launch_bounds__(CTA_THREADS)
fst_gather_kernel(const __grid_constant__ InlineOps inline_ops, const GatherOp *__restrict__ table,
                  unsigned n_ops, uint64_t total_subs) {
    const GatherOp *ops = INLINE ? inline_ops.op : table;
    const unsigned lane = threadIdx.x & 31u;
    const uint64_t warp = (uint64_t)blockIdx.x * WARPS_PER_CTA + (threadIdx.x >> 5);
    const uint64_t step = (uint64_t)gridDim.x * WARPS_PER_CTA * SUBS_PER_WARP_STEP;
    for (uint64_t g = warp * SUBS_PER_WARP_STEP; g < total_subs; g += step) {
        Span s[SUBS_PER_WARP_STEP];
        uint4 v[SUBS_PER_WARP_STEP][VEC_PER_LANE];
#pragma unroll
        for (int u = 0; u < SUBS_PER_WARP_STEP; ++u) {
            if (g + u < total_subs) {
                s[u] = open_sub(ops, n_ops, g + u, lane);
                load_span(s[u], v[u]);
            } else {
                s[u].nvec = 0;
                s[u].glane = 0;
                s[u].glanes = 32;
            }
        }
#pragma unroll
        for (int u = 0; u < SUBS_PER_WARP_STEP; ++u) store_span(s[u], v[u]);
    }
}

// Realign: one span, flat indexing, no op table.  dst + head is 16-byte aligned; the body has
// nvec vectors read at byte offset `shift` inside aligned source words.
constexpr int REALIGN_UNROLL = 4;
__global__ void __launch_bounds__(CTA_THREADS)
fst_realign_kernel(unsigned char *__restrict__ dst, const unsigned char *__restrict__ src,
                   uint64_t nbytes) {
    unsigned head = (16u - (unsigned)((uintptr_t)dst & 15u)) & 15u;
    if (head > nbytes) head = (unsigned)nbytes;
    const uint64_t body = nbytes - head;
    const uint64_t nvec = body >> 4;
    const unsigned tail = (unsigned)(body & 15u);
    if (blockIdx.x == 0) {
        if (threadIdx.x < head) dst[threadIdx.x] = src[threadIdx.x];
        if (threadIdx.x >= 32 && threadIdx.x - 32 < tail) {
            const uint64_t o = head + (nvec << 4) + (threadIdx.x - 32);
            dst[o] = src[o];
        }
    }
    const unsigned char *sb = src + head;
    uint4 *d = reinterpret_cast<uint4 *>(dst + head);
    const unsigned shift = (unsigned)((uintptr_t)sb & 15u);
    const uint4 *s = reinterpret_cast<const uint4 *>(sb - shift);
    // a CTA moves REALIGN_UNROLL consecutive 4 KiB stripes per step (one vector per thread each)
    const uint64_t stride = (uint64_t)gridDim.x * CTA_THREADS * REALIGN_UNROLL;
    for (uint64_t base = (uint64_t)blockIdx.x * CTA_THREADS * REALIGN_UNROLL + threadIdx.x;
         base < nvec; base += stride) {
        uint4 v[REALIGN_UNROLL];
        if (shift == 0) {
#pragma unroll
            for (int j = 0; j < REALIGN_UNROLL; ++j) {
                const uint64_t i = base + (uint64_t)j * CTA_THREADS;
                if (i < nvec) v[j] = ld_stream(s + i);
            }
        } else {
#pragma unroll
            for (int j = 0; j < REALIGN_UNROLL; ++j) {
                const uint64_t i = base + (uint64_t)j * CTA_THREADS;
                if (i < nvec) {
                    const uint4 lo = ld_keep(s + i);
                    const uint4 hi = ld_keep(s + i + 1);
                    v[j] = funnel16(lo, hi, shift);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < REALIGN_UNROLL; ++j) {
            const uint64_t i = base + (uint64_t)j * CTA_THREADS;
            if (i < nvec) st_stream(d + i, v[j]);
        }
    }
}

}  // namespace fst

// ------------------------------------------------------------------------------------------
// Host side: argument checks, op table construction, workspaces, launches
// ------------------------------------------------------------------------------------------
namespace fst {

namespace {

constexpr unsigned TABLE_SLOT_OPS = 16384;  // ops per workspace slot (1 MiB of GatherOp)
constexpr int TABLE_SLOTS = 4;
constexpr int MAX_DEVICES = 64;

// Per-device workspace of the table path: a small ring of (pinned host, device) op tables.  A
// slot is reused only after the event recorded behind the launch that read it has completed.
struct Workspace {
    bool ready = false;
    GatherOp *host_tab[TABLE_SLOTS] = {};
    GatherOp *dev_tab[TABLE_SLOTS] = {};
    cudaEvent_t done[TABLE_SLOTS] = {};
    int next = 0;
    int grid_limit = 0;
};
std::mutex g_ws_mutex;
Workspace g_ws[MAX_DEVICES];
std::atomic<int> g_grid_limit[MAX_DEVICES];  // 0 = not computed yet (reader threads ask too)

// Grid size.  Measured on B200 on the 16 GB benchmark launch (2,328 ops, 7.8 M subs, 1965 MHz):
//   persistent grid of 148 x 4 CTAs striding over the work      5.51 ms
//   148 x 4 x 16 CTAs                                           5.09 ms
//   148 x 4 x 64 CTAs                                           4.94 ms
//   148 x 1024 CTAs (each CTA takes about three steps)          4.87 ms
//   one step per CTA (490 k CTAs)                               5.04 ms
// The hardware block scheduler hands out short CTAs in address order and keeps every SM equally
// loaded; a long grid-stride loop lets CTAs drift apart, and the DRAM pages they touch with
// them.  Beyond ~1000 CTAs per SM the per-CTA start-up (op lookup) begins to show.  So the grid
// is min(steps, SMs x 1024).  FST_B200_GRID_LIMIT overrides the bound for experiments.
constexpr int CTAS_PER_SM_BOUND = 1024;
int grid_limit_for(int dev) {
    if (g_grid_limit[dev].load(std::memory_order_relaxed) == 0) {
        int sms = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
        int limit = sms * CTAS_PER_SM_BOUND;
        if (const char *env = std::getenv("FST_B200_GRID_LIMIT"))
            if (std::atoi(env) > 0) limit = std::atoi(env);
        g_grid_limit[dev].store(limit, std::memory_order_relaxed);
    }
    return g_grid_limit[dev].load(std::memory_order_relaxed);
}

int ensure_workspace(int dev) {
    Workspace &w = g_ws[dev];
    if (w.ready) return FST_OK;
    for (int i = 0; i < TABLE_SLOTS; ++i) {
        cudaError_t e = cudaHostAlloc((void **)&w.host_tab[i], TABLE_SLOT_OPS * sizeof(GatherOp), 0);
        if (e == cudaSuccess) e = cudaMalloc((void **)&w.dev_tab[i], TABLE_SLOT_OPS * sizeof(GatherOp));
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&w.done[i], cudaEventDisableTiming);
        if (e != cudaSuccess) {
            set_error("fst_gather: workspace allocation failed: %s", cudaGetErrorString(e));
            return FST_ENOMEM;
        }
    }
    w.ready = true;
    return FST_OK;
}

// FST_B200_SHORT_ROWS=0 turns the short-row decomposition off (every row its own sub), for
// measurements of what it buys.
bool short_rows_enabled() {
    static const bool on = [] {
        const char *env = std::getenv("FST_B200_SHORT_ROWS");
        return !(env && env[0] == '0');
    }();
    return on;
}

// One caller op as a device record that starts at sub `first_sub`; returns how many subs it has
// (0: nothing to copy, no record written).  A contiguous op collapses to one row.
uint64_t fill_record(fst_copy2d_t c, uint64_t first_sub, GatherOp &g) {
    if (c.rows == 0 || c.row_bytes == 0) return 0;
    if (c.rows > 1 && c.src_pitch == c.row_bytes && c.dst_pitch == c.row_bytes) {
        c.row_bytes *= c.rows;
        c.rows = 1;
    }
    g.src = c.src;
    g.dst = c.dst;
    g.src_pitch = c.rows > 1 ? c.src_pitch : 0;
    g.dst_pitch = c.rows > 1 ? c.dst_pitch : 0;
    g.row_bytes = c.row_bytes;
    g.first_sub = first_sub;
    g.rows = c.rows;
    if (c.rows > 1 && c.row_bytes <= (uint64_t)SHORT_ROW_BYTES && short_rows_enabled()) {
        // lanes per row: the power of two whose registers (LANE_BYTES per lane) hold the row
        uint32_t glanes = 1;
        while ((uint64_t)glanes * LANE_BYTES < c.row_bytes) glanes *= 2;
        const uint64_t rows_per_sub = 32u / glanes;
        g.subs_per_row = 0;
        g.lead = glanes;
        return (c.rows + rows_per_sub - 1) / rows_per_sub;
    }
    g.lead = (g.dst_pitch % 16 == 0) ? (uint32_t)(c.dst & 15u) : 0u;
    // check_ops has refused rows of more than 2^32 subs (8 TiB)
    const uint64_t spr = (c.row_bytes + g.lead + SUB_BYTES - 1) / SUB_BYTES;
    g.subs_per_row = (uint32_t)spr;
    return c.rows * spr;
}

// Device records of all caller ops, with the subs of each record beside them; returns total subs.
uint64_t build_ops(const fst_copy2d_t *in, uint64_t n, std::vector<GatherOp> &out,
                   std::vector<uint64_t> &subs_of, uint64_t &payload) {
    uint64_t subs = 0;
    payload = 0;
    out.clear();
    subs_of.clear();
    out.reserve(n);
    subs_of.reserve(n);
    for (uint64_t i = 0; i < n; ++i) {
        GatherOp g;
        const uint64_t k = fill_record(in[i], subs, g);
        if (k == 0) continue;
        subs += k;
        payload += in[i].rows * in[i].row_bytes;
        out.push_back(g);
        subs_of.push_back(k);
    }
    return subs;
}

int check_ops(const fst_copy2d_t *ops, uint64_t n, uint64_t src_base, uint64_t src_len,
              uint64_t dst_base, uint64_t dst_len) {
    for (uint64_t i = 0; i < n; ++i) {
        const fst_copy2d_t &c = ops[i];
        if (c.rows == 0 || c.row_bytes == 0) continue;
        if (c.src == 0 || c.dst == 0) {
            set_error("fst_gather: op %llu has a null address", (unsigned long long)i);
            return FST_EINVAL;
        }
        if (c.rows > 1 && (c.src_pitch < c.row_bytes || c.dst_pitch < c.row_bytes)) {
            set_error("fst_gather: op %llu: pitch smaller than row_bytes (rows would overlap)",
                      (unsigned long long)i);
            return FST_EINVAL;
        }
        if ((c.row_bytes + 15 + SUB_BYTES - 1) / SUB_BYTES > 0xffffffffull) {
            set_error("fst_gather: op %llu: row_bytes too large", (unsigned long long)i);
            return FST_ELIMIT;
        }
        // end addresses, refusing anything that wraps around 2^64 (a wrapped end would slip
        // past the range checks below)
        uint64_t s_end = 0, d_end = 0;
        if (__builtin_mul_overflow(c.rows - 1, c.src_pitch, &s_end) ||
            __builtin_add_overflow(s_end, c.row_bytes, &s_end) ||
            __builtin_add_overflow(s_end, c.src, &s_end) ||
            __builtin_mul_overflow(c.rows - 1, c.dst_pitch, &d_end) ||
            __builtin_add_overflow(d_end, c.row_bytes, &d_end) ||
            __builtin_add_overflow(d_end, c.dst, &d_end) ||
            (src_len && src_base + src_len < src_base) || (dst_len && dst_base + dst_len < dst_base)) {
            set_error("fst_gather: op %llu: address arithmetic overflows 64 bits",
                      (unsigned long long)i);
            return FST_ERANGE;
        }
        if (src_len && (c.src < src_base || s_end > src_base + src_len)) {
            set_error("fst_gather: op %llu reads [%#llx,%#llx) outside the source buffer "
                      "[%#llx,%#llx)", (unsigned long long)i, (unsigned long long)c.src,
                      (unsigned long long)s_end, (unsigned long long)src_base,
                      (unsigned long long)(src_base + src_len));
            return FST_ERANGE;
        }
        if (dst_len && (c.dst < dst_base || d_end > dst_base + dst_len)) {
            set_error("fst_gather: op %llu writes [%#llx,%#llx) outside the destination buffer "
                      "[%#llx,%#llx)", (unsigned long long)i, (unsigned long long)c.dst,
                      (unsigned long long)d_end, (unsigned long long)dst_base,
                      (unsigned long long)(dst_base + dst_len));
            return FST_ERANGE;
        }
    }
    return FST_OK;
}

unsigned grid_for(uint64_t total_subs, int limit) {
    const uint64_t per_cta = (uint64_t)WARPS_PER_CTA * SUBS_PER_WARP_STEP;
    uint64_t want = (total_subs + per_cta - 1) / per_cta;
    if (want > (uint64_t)limit) want = (uint64_t)limit;
    if (want == 0) want = 1;
    return (unsigned)want;
}

}  // namespace

int launch_realign(void *dst, const void *src, uint64_t nbytes, void *stream) {
    int dev = 0;
    cudaGetDevice(&dev);
    const int limit = grid_limit_for(dev < MAX_DEVICES ? dev : 0);
    const uint64_t per_cta = (uint64_t)CTA_THREADS * REALIGN_UNROLL * 16;
    uint64_t want = (nbytes + per_cta - 1) / per_cta;
    if (want > (uint64_t)limit) want = (uint64_t)limit;
    if (want == 0) want = 1;
    fst_realign_kernel<<<(unsigned)want, CTA_THREADS, 0, (cudaStream_t)stream>>>(
        (unsigned char *)dst, (const unsigned char *)src, nbytes);
    g_counters.kernel_launches.fetch_add(1, std::memory_order_relaxed);
    g_counters.bytes_realigned.fetch_add(nbytes, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}

}  // namespace fst

extern "C" int fst_realign(uint64_t dst, uint64_t src, uint64_t nbytes, uint64_t stream) {
    using namespace fst;
    clear_error();
    if (!cuda_usable()) {
        set_error("fst_realign: no CUDA device");
        return FST_ENOCUDA;
    }
    if (nbytes == 0) return FST_OK;
    if (dst == 0 || src == 0) {
        set_error("fst_realign: null address");
        return FST_EINVAL;
    }
    if (dst < src + nbytes && src < dst + nbytes) {
        set_error("fst_realign: source and destination ranges overlap");
        return FST_EINVAL;
    }
    const int e = launch_realign((void *)dst, (const void *)src, nbytes, (void *)stream);
    if (e != 0) {
        set_error("fst_realign: launch failed: %s", cudaGetErrorString((cudaError_t)e));
        return FST_ECUDA;
    }
    return FST_OK;
}

extern "C" int fst_gather(const fst_copy2d_t *ops, uint64_t n_ops, uint64_t src_base,
                          uint64_t src_len, uint64_t dst_base, uint64_t dst_len,
                          uint64_t stream) {
    return fst_gather_limited(ops, n_ops, src_base, src_len, dst_base, dst_len, stream, 0);
}

extern "C" int fst_gather_limited(const fst_copy2d_t *ops, uint64_t n_ops, uint64_t src_base,
                                  uint64_t src_len, uint64_t dst_base, uint64_t dst_len,
                                  uint64_t stream, uint32_t max_ctas) {
    using namespace fst;
    clear_error();
    if (!cuda_usable()) {
        set_error("fst_gather: no CUDA device");
        return FST_ENOCUDA;
    }
    if (n_ops == 0) return FST_OK;
    if (ops == nullptr) {
        set_error("fst_gather: ops is null");
        return FST_EINVAL;
    }
    int rc = check_ops(ops, n_ops, src_base, src_len, dst_base, dst_len);
    if (rc != FST_OK) return rc;

    std::vector<GatherOp> recs;
    std::vector<uint64_t> subs_of;
    uint64_t payload = 0;
    build_ops(ops, n_ops, recs, subs_of, payload);
    if (recs.empty()) return FST_OK;

    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= MAX_DEVICES) {
        set_error("fst_gather: device index %d not supported", dev);
        return FST_ELIMIT;
    }
    cudaStream_t st = (cudaStream_t)stream;
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    int limit = grid_limit_for(dev);
    if (max_ctas > 0 && (int)max_ctas < limit) limit = (int)max_ctas;

    size_t pos = 0;
    while (pos < recs.size()) {
        const size_t left = recs.size() - pos;
        if (left <= FST_GATHER_INLINE_OPS) {
            InlineOps p;
            std::memset(&p, 0, sizeof(p));
            const uint64_t base = recs[pos].first_sub;
            uint64_t subs = 0;
            for (size_t i = 0; i < left; ++i) {
                p.op[i] = recs[pos + i];
                p.op[i].first_sub -= base;
                subs += subs_of[pos + i];
            }
            fst_gather_kernel<true><<<grid_for(subs, limit), CTA_THREADS, 0, st>>>(
                p, nullptr, (unsigned)left, subs);
            pos += left;
        } else {
            rc = ensure_workspace(dev);
            if (rc != FST_OK) return rc;
            Workspace &w = g_ws[dev];
            const int slot = w.next;
            w.next = (w.next + 1) % TABLE_SLOTS;
            cudaError_t e = cudaEventSynchronize(w.done[slot]);
            if (e != cudaSuccess) {
                set_error("fst_gather: waiting for a workspace slot failed: %s",
                          cudaGetErrorString(e));
                return FST_ECUDA;
            }
            const size_t take = std::min<size_t>(left, TABLE_SLOT_OPS);
            const uint64_t base = recs[pos].first_sub;
            uint64_t subs = 0;
            for (size_t i = 0; i < take; ++i) {
                w.host_tab[slot][i] = recs[pos + i];
                w.host_tab[slot][i].first_sub -= base;
                subs += subs_of[pos + i];
            }
            e = cudaMemcpyAsync(w.dev_tab[slot], w.host_tab[slot], take * sizeof(GatherOp),
                                cudaMemcpyHostToDevice, st);
            if (e != cudaSuccess) {
                set_error("fst_gather: op table upload failed: %s", cudaGetErrorString(e));
                return FST_ECUDA;
            }
            InlineOps none;
            std::memset(&none, 0, sizeof(none));
            fst_gather_kernel<false><<<grid_for(subs, limit), CTA_THREADS, 0, st>>>(
                none, w.dev_tab[slot], (unsigned)take, subs);
            cudaEventRecord(w.done[slot], st);
            pos += take;
        }
        g_counters.kernel_launches.fetch_add(1, std::memory_order_relaxed);
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) {
            set_error("fst_gather: launch failed: %s", cudaGetErrorString(e));
            return FST_ECUDA;
        }
    }
    g_counters.bytes_gathered.fetch_add(payload, std::memory_order_relaxed);
    return FST_OK;
}

extern "C" int fst_release_workspaces(void) {
    using namespace fst;
    if (!cuda_usable()) return FST_OK;
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    int cur = 0;
    cudaGetDevice(&cur);
    for (int d = 0; d < MAX_DEVICES; ++d) {
        Workspace &w = g_ws[d];
        if (!w.ready) continue;
        cudaSetDevice(d);
        for (int i = 0; i < TABLE_SLOTS; ++i) {
            cudaEventSynchronize(w.done[i]);
            cudaEventDestroy(w.done[i]);
            cudaFree(w.dev_tab[i]);
            cudaFreeHost(w.host_tab[i]);
        }
        w = Workspace();
    }
    cudaSetDevice(cur);
    return FST_OK;
}

// ------------------------------------------------------------------------------------------
// fst_gather_static: the gather for callers that cannot allocate
// ------------------------------------------------------------------------------------------
namespace fst {
namespace {

// The op table of fst_gather_static.  Part of the library image: every GPU that loads the
// library holds these 256 KiB until the process exits.  In host code this name is only a
// handle for cudaGetSymbolAddress, never an address a kernel may be given.
static __device__ __align__(256) GatherOp g_static_table[FST_GATHER_STATIC_MAX_OPS];

// Host-side twin in which the records are assembled (fixed storage, no heap), and the device
// address of the table per device (looked up once, with that device current).
GatherOp g_static_host[FST_GATHER_STATIC_MAX_OPS];
GatherOp *g_static_dev[MAX_DEVICES];
// Guards the host twin and the address cache.  Its own lock, not the workspace's: the table
// upload below can stall the calling thread until earlier work on the stream is done, and
// fst_gather callers on other threads must not queue behind that.
std::mutex g_static_mutex;

}  // namespace
}  // namespace fst

extern "C" int fst_gather_static(const fst_copy2d_t *ops, uint64_t n_ops, uint64_t src_base,
                                 uint64_t src_len, uint64_t dst_base, uint64_t dst_len,
                                 uint64_t stream) {
    using namespace fst;
    clear_error();
    if (!cuda_usable()) {
        set_error("fst_gather_static: no CUDA device");
        return FST_ENOCUDA;
    }
    if (n_ops == 0) return FST_OK;
    if (ops == nullptr) {
        set_error("fst_gather_static: ops is null");
        return FST_EINVAL;
    }
    if (n_ops > FST_GATHER_STATIC_MAX_OPS) {
        set_error("fst_gather_static: %llu ops exceed the fixed table of %d; split the request",
                  (unsigned long long)n_ops, FST_GATHER_STATIC_MAX_OPS);
        return FST_ELIMIT;
    }
    int rc = check_ops(ops, n_ops, src_base, src_len, dst_base, dst_len);
    if (rc != FST_OK) return rc;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= MAX_DEVICES) {
        set_error("fst_gather_static: device index %d not supported", dev);
        return FST_ELIMIT;
    }
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (g_static_dev[dev] == nullptr) {
        GatherOp *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void **)&p, g_static_table);
        if (e != cudaSuccess || p == nullptr) {
            (void)cudaGetLastError();
            set_error("fst_gather_static: cudaGetSymbolAddress failed on device %d: %s", dev,
                      cudaGetErrorString(e));
            return FST_ECUDA;
        }
        g_static_dev[dev] = p;
    }
    // build the records in the fixed host twin (same rules as fst_gather's table)
    unsigned count = 0;
    uint64_t subs = 0, payload = 0;
    for (uint64_t i = 0; i < n_ops; ++i) {
        const uint64_t k = fill_record(ops[i], subs, g_static_host[count]);
        if (k == 0) continue;
        ++count;
        subs += k;
        payload += ops[i].rows * ops[i].row_bytes;
    }
    if (count == 0) return FST_OK;
    cudaStream_t st = (cudaStream_t)stream;
    GatherOp *table = g_static_dev[dev];
    cudaError_t e = cudaMemcpyAsync(table, g_static_host, count * sizeof(GatherOp),
                                    cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) {
        set_error("fst_gather_static: op table upload failed: %s", cudaGetErrorString(e));
        return FST_ECUDA;
    }
    InlineOps none;
    std::memset(&none, 0, sizeof(none));
    fst_gather_kernel<false><<<grid_for(subs, grid_limit_for(dev)), CTA_THREADS, 0, st>>>(
        none, table, count, subs);
    e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("fst_gather_static: launch failed: %s", cudaGetErrorString(e));
        return FST_ECUDA;
    }
    g_counters.kernel_launches.fetch_add(1, std::memory_order_relaxed);
    g_counters.bytes_gathered.fetch_add(payload, std::memory_order_relaxed);
    return FST_OK;
}

// ------------------------------------------------------------------------------------------
// fst_convert: narrowing floating-point conversion of many tensors in one launch
// ------------------------------------------------------------------------------------------
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace fst {

// Device record of one conversion (64 bytes, so that it can share the gather's op-table ring).
struct ConvertOp {
    uint64_t src;
    uint64_t dst;
    uint64_t n;            // elements
    uint64_t first_chunk;  // chunks of CONVERT_CHUNK elements in earlier ops
    uint32_t src_t;
    uint32_t dst_t;
    uint64_t pad[3];
};
static_assert(sizeof(ConvertOp) == sizeof(GatherOp), "ConvertOp shares the GatherOp table ring");

constexpr unsigned CONVERT_CHUNK = 4096;  // elements one warp converts per step (128 per lane)

__device__ __forceinline__ float load_as_float(const void *p, uint32_t t, uint64_t i) {
    switch (t) {
        case FST_DT_F64: return (float)reinterpret_cast<const double *>(p)[i];
        case FST_DT_F32: return reinterpret_cast<const float *>(p)[i];
        case FST_DT_F16: return __half2float(reinterpret_cast<const __half *>(p)[i]);
        default: return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
    }
}

__device__ __forceinline__ void store_from_float(void *p, uint32_t t, uint64_t i, float v) {
    switch (t) {
        case FST_DT_F32: reinterpret_cast<float *>(p)[i] = v; break;
        case FST_DT_F16: reinterpret_cast<__half *>(p)[i] = __float2half_rn(v); break;
        default: reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v); break;
    }
}

// One warp per chunk; lanes take interleaved groups of 4 elements so that a warp instruction
// touches one contiguous run.  F32 -> 16-bit with aligned addresses moves 16-byte loads and
// 8-byte stores; every other case goes element by element (still coalesced).
__global__ void __launch_bounds__(CTA_THREADS)
fst_convert_kernel(const ConvertOp *__restrict__ ops, unsigned n_ops, uint64_t total_chunks) {
    const unsigned lane = threadIdx.x & 31u;
    const uint64_t warp = (uint64_t)blockIdx.x * WARPS_PER_CTA + (threadIdx.x >> 5);
    const uint64_t step = (uint64_t)gridDim.x * WARPS_PER_CTA;
    for (uint64_t c = warp; c < total_chunks; c += step) {
        unsigned lo = 0, hi = n_ops;
        while (hi - lo > 1) {
            const unsigned mid = (lo + hi) >> 1;
            if (ops[mid].first_chunk <= c) lo = mid; else hi = mid;
        }
        const ConvertOp &op = ops[lo];
        const uint64_t beg = (c - op.first_chunk) * CONVERT_CHUNK;
        const uint64_t end = beg + CONVERT_CHUNK < op.n ? beg + CONVERT_CHUNK : op.n;
        const void *s = reinterpret_cast<const void *>(op.src);
        void *d = reinterpret_cast<void *>(op.dst);
        const bool fast = op.src_t == FST_DT_F32 && (op.dst_t == FST_DT_F16 || op.dst_t == FST_DT_BF16) &&
                          ((op.src & 15u) == 0) && ((op.dst & 7u) == 0);
        if (fast) {
            const float4 *s4 = reinterpret_cast<const float4 *>(s);
            uint2 *d4 = reinterpret_cast<uint2 *>(d);
            const uint64_t g_end = end >> 2;
            for (uint64_t g = (beg >> 2) + lane; g < g_end; g += 32) {
                const float4 v = __ldcs(s4 + g);
                uint2 o;
                if (op.dst_t == FST_DT_F16) {
                    const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
                    o.x = *reinterpret_cast<const unsigned *>(&a);
                    o.y = *reinterpret_cast<const unsigned *>(&b);
                } else {
                    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
                    o.x = *reinterpret_cast<const unsigned *>(&a);
                    o.y = *reinterpret_cast<const unsigned *>(&b);
                }
                __stcs(d4 + g, o);
            }
            for (uint64_t i = (g_end << 2) + lane; i < end; i += 32)   // ragged tail of the tensor
                store_from_float(d, op.dst_t, i, load_as_float(s, op.src_t, i));
        } else {
            for (uint64_t i = beg + lane; i < end; i += 32)
                store_from_float(d, op.dst_t, i, load_as_float(s, op.src_t, i));
        }
    }
}

}  // namespace fst

extern "C" int fst_convert(const fst_convert_op_t *ops, uint64_t n_ops, uint64_t stream) {
    using namespace fst;
    clear_error();
    if (!cuda_usable()) {
        set_error("fst_convert: no CUDA device");
        return FST_ENOCUDA;
    }
    if (n_ops == 0) return FST_OK;
    if (ops == nullptr) {
        set_error("fst_convert: ops is null");
        return FST_EINVAL;
    }
    static const unsigned width[4] = {8, 4, 2, 2};
    std::vector<ConvertOp> recs;
    recs.reserve(n_ops);
    uint64_t chunks = 0;
    for (uint64_t i = 0; i < n_ops; ++i) {
        const fst_convert_op_t &c = ops[i];
        if (c.n_elements == 0) continue;
        if (c.src == 0 || c.dst == 0 || c.src_dtype < 0 || c.src_dtype > 3 || c.dst_dtype < 1 ||
            c.dst_dtype > 3) {
            set_error("fst_convert: op %llu: bad address or dtype code", (unsigned long long)i);
            return FST_EINVAL;
        }
        if (width[c.dst_dtype] > width[c.src_dtype]) {
            set_error("fst_convert: op %llu widens (%d -> %d); only narrowing or same-width "
                      "conversions are supported", (unsigned long long)i, c.src_dtype, c.dst_dtype);
            return FST_EINVAL;
        }
        if (c.src % width[c.src_dtype] || c.dst % width[c.dst_dtype]) {
            set_error("fst_convert: op %llu: address not aligned to its element size",
                      (unsigned long long)i);
            return FST_EINVAL;
        }
        const uint64_t s_end = c.src + c.n_elements * width[c.src_dtype];
        const uint64_t d_end = c.dst + c.n_elements * width[c.dst_dtype];
        if (c.dst < s_end && c.src < d_end) {
            set_error("fst_convert: op %llu: source and destination overlap", (unsigned long long)i);
            return FST_EINVAL;
        }
        ConvertOp r = {};
        r.src = c.src;
        r.dst = c.dst;
        r.n = c.n_elements;
        r.src_t = (uint32_t)c.src_dtype;
        r.dst_t = (uint32_t)c.dst_dtype;
        r.first_chunk = chunks;
        chunks += (c.n_elements + CONVERT_CHUNK - 1) / CONVERT_CHUNK;
        recs.push_back(r);
    }
    if (recs.empty()) return FST_OK;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= MAX_DEVICES) {
        set_error("fst_convert: device index %d not supported", dev);
        return FST_ELIMIT;
    }
    cudaStream_t st = (cudaStream_t)stream;
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    int rc = ensure_workspace(dev);
    if (rc != FST_OK) return rc;
    const int limit = grid_limit_for(dev);
    Workspace &w = g_ws[dev];
    size_t pos = 0;
    while (pos < recs.size()) {
        const size_t take = std::min<size_t>(recs.size() - pos, TABLE_SLOT_OPS);
        const int slot = w.next;
        w.next = (w.next + 1) % TABLE_SLOTS;
        cudaError_t e = cudaEventSynchronize(w.done[slot]);
        ConvertOp *host = reinterpret_cast<ConvertOp *>(w.host_tab[slot]);
        const uint64_t base = recs[pos].first_chunk;
        uint64_t n_chunks = 0;
        for (size_t i = 0; i < take; ++i) {
            host[i] = recs[pos + i];
            host[i].first_chunk -= base;
            n_chunks += (recs[pos + i].n + CONVERT_CHUNK - 1) / CONVERT_CHUNK;
        }
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(w.dev_tab[slot], host, take * sizeof(ConvertOp), cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) {
            set_error("fst_convert: op table upload failed: %s", cudaGetErrorString(e));
            return FST_ECUDA;
        }
        uint64_t want = (n_chunks + WARPS_PER_CTA - 1) / WARPS_PER_CTA;
        if (want > (uint64_t)limit) want = (uint64_t)limit;
        fst_convert_kernel<<<(unsigned)want, CTA_THREADS, 0, st>>>(
            reinterpret_cast<const ConvertOp *>(w.dev_tab[slot]), (unsigned)take, n_chunks);
        cudaEventRecord(w.done[slot], st);
        e = cudaGetLastError();
        if (e != cudaSuccess) {
            set_error("fst_convert: launch failed: %s", cudaGetErrorString(e));
            return FST_ECUDA;
        }
        g_counters.kernel_launches.fetch_add(1, std::memory_order_relaxed);
        pos += take;
    }
    return FST_OK;
}
