// Host side of the library: the index state machine (what TurboQuantIndex / IdMapIndex own in the
// reference, turbovec/src/lib.rs:295-401 and id_map.rs:221-272) with the code array, the scales and all
// scratch resident in device memory, and the C ABI declared in include/turbovec_b200.h.
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <shared_mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../../include/turbovec_b200.h"
#include "host_tables.hpp"
#include "ingest.cuh"
#include "io_v7.hpp"
#include "search.cuh"
#include "tv_common.cuh"

namespace {

using namespace tv;

thread_local std::string g_create_error;

template <typename T>
struct DeviceArray {
    T *ptr = nullptr;
    size_t cap = 0;   // elements
    ~DeviceArray() { release(); }
    void release() {
        if (ptr) cudaFree(ptr);
        ptr = nullptr;
        cap = 0;
    }
    // Grows without preserving contents.
    cudaError_t reserve(size_t n) {
        if (n <= cap) return cudaSuccess;
        release();
        cudaError_t e = cudaMalloc(&ptr, std::max<size_t>(n, 1) * sizeof(T));
        if (e == cudaSuccess) cap = n;
        return e;
    }
};

template <typename T>
struct PinnedArray {
    T *ptr = nullptr;
    size_t cap = 0;
    ~PinnedArray() { if (ptr) cudaFreeHost(ptr); }
    cudaError_t reserve(size_t n) {
        if (n <= cap) return cudaSuccess;
        if (ptr) cudaFreeHost(ptr);
        ptr = nullptr; cap = 0;
        cudaError_t e = cudaMallocHost(&ptr, std::max<size_t>(n, 1) * sizeof(T));
        if (e == cudaSuccess) cap = n;
        return e;
    }
};

struct DeviceFlags {        // one pinned + one device copy of the status words of a call
    unsigned long long first_invalid;
    unsigned long long n_allowed;
    unsigned long long first_unknown;   // smallest allowlist index whose id the device table does not hold
    uint32_t n_live;
    uint32_t overflow;
    uint32_t error;
    uint32_t k_eff;
};

// CUDA events around the launches of the dominant kernel (scan, ingest) of one call.
struct Marks {
    std::vector<cudaEvent_t> pool;
    size_t used = 0;
    float total_ms = 0.f;
    int launches = 0;
    ~Marks() { for (cudaEvent_t e : pool) cudaEventDestroy(e); }
    void begin(cudaStream_t st) {
        if (used + 2 > pool.size()) {
            for (int i = 0; i < 64; ++i) {
                cudaEvent_t e;
                if (cudaEventCreate(&e) != cudaSuccess) return;
                pool.push_back(e);
            }
        }
        cudaEventRecord(pool[used], st);
    }
    void end(cudaStream_t st) {
        if (used + 2 > pool.size()) return;
        cudaEventRecord(pool[used + 1], st);
        used += 2;
    }
    // after the stream has been synchronised: total time and count of the bracketed launches
    void collect() {
        float total = 0.f;
        for (size_t i = 0; i + 1 < used; i += 2) {
            float ms = 0.f;
            if (cudaEventElapsedTime(&ms, pool[i], pool[i + 1]) == cudaSuccess) total += ms;
        }
        total_ms = total;
        launches = int(used / 2);
        used = 0;
    }
};

// Everything one search call owns while it runs: a stream, status words, events and the scratch arrays
// (grown on demand, reused).  A handle keeps a small pool of these so that searches from several host threads
// overlap on the device, as the reference's `search(&self)` may run concurrently (turbovec/src/lib.rs:22-52).
struct SearchCtx {
    bool busy = false;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    Marks marks;
    DeviceFlags *d_flags = nullptr;
    DeviceFlags *h_flags = nullptr;
    DeviceArray<float> d_stage;              // query upload
    DeviceArray<float> d_qrot, d_qscale, d_qbias;
    DeviceArray<uint8_t> d_luts;
    DeviceArray<int8_t> d_weights;
    DeviceArray<uint32_t> d_wfrag;
    DeviceArray<uint64_t> d_mask;
    DeviceArray<uint8_t> d_mask_bool;
    DeviceArray<uint32_t> d_slots_in, d_live;
    DeviceArray<uint64_t> d_allow_ids;       // an allowlist resolved on the device
    DeviceArray<uint64_t> d_cand, d_thr, d_topk, d_floor, d_keys_all;
    DeviceArray<uint32_t> d_cnt;
    DeviceArray<float> d_scores;
    DeviceArray<int64_t> d_slots;
    DeviceArray<uint64_t> d_keys_tmp;        // staging of tv_search_device_keys when the shard holds fewer than k vectors
    PinnedArray<float> h_scores;
    PinnedArray<int64_t> h_slots;
    cudaError_t init() {
        cudaError_t e = cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaEventCreate(&ev0);
        if (e == cudaSuccess) e = cudaEventCreate(&ev1);
        if (e == cudaSuccess) e = cudaMalloc(&d_flags, sizeof(DeviceFlags));
        if (e == cudaSuccess) e = cudaMallocHost(&h_flags, sizeof(DeviceFlags));
        // the event pool of the common schedules up front, so that a search creates nothing
        for (int i = 0; i < 64 && e == cudaSuccess; ++i) {
            cudaEvent_t ev;
            e = cudaEventCreate(&ev);
            if (e == cudaSuccess) marks.pool.push_back(ev);
        }
        return e;
    }
    ~SearchCtx() {
        if (stream) cudaStreamSynchronize(stream);
        if (d_flags) cudaFree(d_flags);
        if (h_flags) cudaFreeHost(h_flags);
        if (ev0) cudaEventDestroy(ev0);
        if (ev1) cudaEventDestroy(ev1);
        if (stream) cudaStreamDestroy(stream);
    }
};
constexpr int kSearchCtxs = 2;

// Device copy of the id -> slot table, kept for large allowlists (search.cu: idtab_*_kernel).  The host tables stay the
// authority; this copy is brought up to date lazily, by the first allowlist search after a change.
struct DeviceIdTable {
    DeviceArray<uint64_t> keys;
    DeviceArray<uint32_t> vals;
    int log2cap = 0;
    size_t used = 0;                  // occupied places, tombstones included
    bool valid = false;               // holds slot_to_id as of the last change, minus `pending`
    bool unusable = false;            // an id equal to one of the two marker keys was added: the host path serves everything
    std::vector<std::pair<uint64_t, uint32_t>> pending;   // (id, slot) in order; slot 0xffffffff = removed
    DeviceArray<uint64_t> d_ids;      // staging of a rebuild / an update
    DeviceArray<uint32_t> d_slots;
    cudaEvent_t ev = nullptr;         // recorded after every update; lookups on other streams wait for it
    std::mutex mu;
    ~DeviceIdTable() { if (ev) cudaEventDestroy(ev); }
    void note(uint64_t id, uint32_t slot, size_t n_ids) {
        if (id >= 0xfffffffffffffffeull) unusable = true;
        if (!valid) return;
        pending.emplace_back(id, slot);
        if (pending.size() > n_ids / 4 + 65536) { valid = false; pending.clear(); }   // a rebuild is cheaper
    }
    void reset(const std::vector<uint64_t> &ids) {                  // the whole id table was replaced
        valid = false; pending.clear(); unusable = false;
        for (uint64_t id : ids) if (id >= 0xfffffffffffffffeull) unusable = true;
    }
};
constexpr size_t kDeviceAllowlistMin = 32768;   // allowlists at least this long are resolved on the device

// The index as int8 levels (scan_tc_dense.cu): rows [0, rows_valid) minus the blocks in `dirty` are current.  Built and
// brought up to date lazily by the first large-batch permute-dot search after a change; dropped when the code array moves.
struct ExpandedCopy {
    DeviceArray<int8_t> levels;       // rows_cap x pitch
    size_t rows_cap = 0;              // rows allocated (the capacity of the code array, whole blocks)
    size_t rows_valid = 0;
    int pitch = 0;
    std::vector<uint32_t> dirty;      // blocks below rows_valid whose codes changed in place
    DeviceArray<uint32_t> d_dirty;
    size_t refused_at_cap = 0;        // the allocation for this capacity did not fit: do not try again until it changes
    cudaEvent_t ev = nullptr;         // recorded after every update; searches on other streams wait for it
    std::mutex mu;
    ~ExpandedCopy() { if (ev) cudaEventDestroy(ev); }
    void touch(size_t slot) {         // the codes of `slot` changed in place
        if (slot >= rows_valid) return;
        const uint32_t blk = uint32_t(slot / 32);
        if (!dirty.empty() && dirty.back() == blk) return;
        if (dirty.size() >= 4096) { rows_valid = std::min(rows_valid, size_t(*std::min_element(dirty.begin(), dirty.end())) * 32); dirty.clear(); }
        if (slot < rows_valid) dirty.push_back(blk);
    }
    void shrink(size_t n) { rows_valid = std::min(rows_valid, n); }
    void reset() { rows_valid = 0; dirty.clear(); }
    void drop() { levels.release(); rows_cap = 0; refused_at_cap = 0; reset(); }
};

// An allow-mask kept on the device between searches (tv_mask_prepare_*): words, live-block list and the two
// counts the kernels read.  Any change of the index invalidates it.
struct PreparedMask {
    bool valid = false;
    DeviceArray<uint64_t> words;
    DeviceArray<uint32_t> live;
    DeviceArray<unsigned long long> counts;  // [0] = allowed slots, [1] low word = live blocks
};

}  // namespace

struct tv_index {
    int kind = TV_KIND_POSITIONAL;
    int bits = 4;
    int device = 0;
    size_t dim = 0;          // 0 = lazy
    size_t n = 0;
    int ngroups = 0;
    int sm_count = 148;
    size_t smem_limit = 0;

    // Readers and writers: searches hold the lock shared and take a SearchCtx from the pool; every call that changes
    // the index, and the accessors that use the handle's own stream, hold it exclusively.
    std::shared_mutex mu;
    std::mutex stat_mu;          // error text / detail and the timing figures of the last call
    std::string last_error;
    size_t err_vec = 0, err_coord = 0;
    float err_value = 0.f;
    uint64_t err_id = 0;

    // options
    int score_mode = TV_SCORE_AUTO;
    int64_t mma_min_batch = -1;  // -1: measured switch points (permute-dot 33 queries, u8-LUT 8); 0 never; else as set
    int force_careful = 0;
    int pd_split = 1;            // 1: the small-batch permute-dot scan uses the split level lookup where the codebook allows it
    int ingest_pipeline = 1;     // 1: whole code blocks of an uncalibrated add go through the pipelined ingest kernel
    int tc_tiles = 1;            // accumulator tiles per B slab in the tcgen05 scan (1 or 2); 1 measured faster
    int small_scan = 5;          // permute-dot scan for up to 16 queries: -1 = scan_pd_kernel, else a scan_small_kernel variant
                                 // (5 = four-stage rings, two CTAs per SM, swizzled tensor copies: the fastest measured)
    int tc_wide = 1;             // 1: batches above 256 queries share every expanded code slab between two query groups
    int tc_expanded = 1;         // 1: large permute-dot batches scan an int8 copy of the index when device memory has room for it; 0 never; 2 always (fail if it does not fit)
    int dense_pair = 1;          // 1: the scan over the int8 copy runs on CTA pairs (cta_group::2)
    int fail_next = 0;           // test hook (TV_OPT_FAIL_NEXT): the next device allocation / upload of a call reports failure

    cudaStream_t stream = nullptr;           // mutations and accessors
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    cudaEvent_t ev_mut = nullptr;            // recorded on `stream` after every mutation; searches wait for it
    std::atomic<uint64_t> launches{0};
    float last_ms = 0.f;
    Marks marks;                             // ingest launches of the last add
    float last_main_ms = 0.f;
    int last_main_launches = 0;

    // tables (host + device)
    bool tables_ready = false;
    RotationTables rot;
    Codebook cb;
    std::vector<float> shift, scale_tq;      // empty = uncalibrated
    DeviceArray<uint16_t> d_perm;            // [2][dim]
    DeviceArray<float> d_codebook;           // boundaries (16 slots) then centroids (16 slots)
    DeviceArray<uint2> d_qgrid;              // quantisation grid of the pipelined ingest kernel
    QuantGrid qgrid;                         // cells == nullptr: the codebook has no valid grid
    DeviceArray<uint8_t> d_store_bank;       // exchange layout of the pipelined ingest kernel (empty: plain rows)
    DeviceArray<uint16_t> d_perm1_exchange;
    bool exchange_ready = false;
    DeviceArray<float> d_calib;              // shift, scale, inv_scale  [3][dim]
    float level_scale = 1.f;                 // cs of the permute-dot level table
    int8_t levels[16] = {0};

    // storage
    uint8_t *d_codes = nullptr;
    size_t code_blocks_cap = 0;
    float *d_scales = nullptr;
    size_t scales_cap = 0;

    // scratch of the mutating calls
    DeviceArray<float> d_stage;              // ingest staging (calibration sample)
    DeviceArray<uint8_t> d_row;              // one row's byte-groups (get_row / set_row)
    // host-memory adds: two pinned + two device staging buffers, a copy stream and per-buffer events
    PinnedArray<float> h_add[2];
    DeviceArray<float> d_add[2];
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t ev_copied[2] = {nullptr, nullptr}, ev_consumed[2] = {nullptr, nullptr};
    DeviceFlags *d_flags = nullptr;
    DeviceFlags *h_flags = nullptr;

    // search contexts
    SearchCtx ctx[kSearchCtxs];
    std::mutex ctx_mu;
    std::condition_variable ctx_cv;
    PreparedMask prepared;
    DeviceIdTable idtab;
    ExpandedCopy expanded;

    // id map (ids never reach the device; id_map.rs:221-272)
    std::vector<uint64_t> slot_to_id;
    std::unordered_map<uint64_t, uint32_t> id_to_slot;

    // binding to the file last synced to or loaded from (lib.rs:364-400)
    bool sync_bound = false;
    std::string sync_path;
    V7Cursor sync_cursor;
    std::unordered_set<size_t> sync_pending;   // slots whose redo ops ride the committed header
    std::unordered_set<size_t> sync_fresh;     // committed slots dirtied since that commit
    uint64_t calib_gen = 0;                    // bumped by every committed calibration
    void mark_dirty(size_t slot) {             // lib.rs:1575-1579
        if (sync_bound && slot < size_t(sync_cursor.n_synced) / kBlock * kBlock) sync_fresh.insert(slot);
    }

    ~tv_index() {
        cudaSetDevice(device);
        if (stream) cudaStreamSynchronize(stream);
        if (d_codes) cudaFree(d_codes);
        if (d_scales) cudaFree(d_scales);
        if (d_flags) cudaFree(d_flags);
        if (h_flags) cudaFreeHost(h_flags);
        if (ev0) cudaEventDestroy(ev0);
        if (ev1) cudaEventDestroy(ev1);
        if (ev_mut) cudaEventDestroy(ev_mut);
        for (int b = 0; b < 2; ++b) {
            if (ev_copied[b]) cudaEventDestroy(ev_copied[b]);
            if (ev_consumed[b]) cudaEventDestroy(ev_consumed[b]);
        }
        if (copy_stream) cudaStreamDestroy(copy_stream);
        if (stream) cudaStreamDestroy(stream);
    }
};

namespace {

int fail(tv_index *h, int code, const std::string &msg) {
    if (h) {
        std::lock_guard<std::mutex> g(h->stat_mu);
        h->last_error = msg;
    } else {
        g_create_error = msg;
    }
    return code;
}

// Brackets one ingest launch with two events from the handle's pool.
void mark_begin(tv_index *h) { h->marks.begin(h->stream); }
void mark_end(tv_index *h) { h->marks.end(h->stream); }
void collect_marks(tv_index *h) {
    h->marks.collect();
    h->last_main_ms = h->marks.total_ms;
    h->last_main_launches = h->marks.launches;
}

// Called at the end of every call that changed device state on the handle's stream: searches run on their own
// streams and wait for this event first.  Also drops a prepared mask, which describes the index as it was.
void mutation_done(tv_index *h) {
    cudaEventRecord(h->ev_mut, h->stream);
    h->prepared.valid = false;
}

// Test hook: with TV_OPT_FAIL_NEXT set, the next guarded allocation or upload of a call reports
// cudaErrorMemoryAllocation instead of running, once.
cudaError_t injected_failure(tv_index *h) {
    if (h->fail_next > 0 && --h->fail_next == 0) return cudaErrorMemoryAllocation;
    return cudaSuccess;
}

#define TV_CUDA(expr)                                                                              \
    do {                                                                                           \
        cudaError_t e__ = (expr);                                                                  \
        if (e__ != cudaSuccess) {                                                                  \
            cudaGetLastError();                                                                    \
            return fail(h, e__ == cudaErrorMemoryAllocation ? TV_ERR_OUT_OF_MEMORY : TV_ERR_CUDA,  \
                        std::string(#expr) + ": " + cudaGetErrorString(e__));                      \
        }                                                                                          \
    } while (0)

int resolve_mode(const tv_index *h) {
    const int vm = (h->ngroups % 4) == 0;
    int m = h->score_mode;
    if (m == TV_SCORE_AUTO) m = (vm && h->bits == 4) ? TV_SCORE_PERMUTE_DOT : (vm ? TV_SCORE_LUT_MULADD : TV_SCORE_LUT_FLUSH);
    if (m == TV_SCORE_PERMUTE_DOT && h->bits != 4) m = TV_SCORE_LUT_MULADD;
    return m;
}

// Uploads h->cb and derives the permute-dot level table from it.
int upload_codebook(tv_index *h) {
    float cbuf[32] = {0};
    for (size_t i = 0; i < h->cb.boundaries.size(); ++i) cbuf[i] = h->cb.boundaries[i];
    for (size_t i = 0; i < h->cb.centroids.size(); ++i) cbuf[16 + i] = h->cb.centroids[i];
    TV_CUDA(h->d_codebook.reserve(32));
    TV_CUDA(cudaMemcpyAsync(h->d_codebook.ptr, cbuf, sizeof cbuf, cudaMemcpyHostToDevice, h->stream));
    QuantGridHost grid;
    h->qgrid = QuantGrid{};
    if (build_quant_grid(h->cb.boundaries.data(), int(h->cb.boundaries.size()), grid)) {
        static_assert(sizeof(QuantCell) == sizeof(uint2), "grid cells are uploaded as they are");
        TV_CUDA(h->d_qgrid.reserve(grid.cells.size()));
        TV_CUDA(cudaMemcpyAsync(h->d_qgrid.ptr, grid.cells.data(), grid.cells.size() * sizeof(uint2), cudaMemcpyHostToDevice, h->stream));
        h->qgrid.cells = h->d_qgrid.ptr; h->qgrid.a = grid.a; h->qgrid.b = grid.b;
    }
    TV_CUDA(cudaStreamSynchronize(h->stream));
    if (h->bits == 4) {
        // search.rs:2812-2819: cs = cmax/127, level = clamp(round(c/cs), +-127)
        float cmax = 0.f;
        for (float c : h->cb.centroids) cmax = std::fmax(cmax, std::fabs(c));
        const float cs = cmax > 0.f ? cmax / 127.0f : 1.0f;
        for (int i = 0; i < 16; ++i) {
            float r = std::round(h->cb.centroids[i] / cs);
            r = std::fmin(std::fmax(r, -127.0f), 127.0f);
            h->levels[i] = int8_t(int(r));
        }
        h->level_scale = cs;
    }
    return TV_OK;
}

// Builds rotation tables, codebook and the permute-dot level table for the (now fixed) dimension.
int ensure_tables(tv_index *h) {
    if (h->tables_ready) return TV_OK;
    const int dim = int(h->dim);
    h->ngroups = dim / (8 / h->bits);
    h->rot = build_rotation_tables(dim);
    h->cb = codebook(h->bits, dim);
    TV_CUDA(h->d_perm.reserve(size_t(2) * dim));
    TV_CUDA(cudaMemcpyAsync(h->d_perm.ptr, h->rot.packed[0].data(), size_t(dim) * 2, cudaMemcpyHostToDevice, h->stream));
    TV_CUDA(cudaMemcpyAsync(h->d_perm.ptr + dim, h->rot.packed[1].data(), size_t(dim) * 2, cudaMemcpyHostToDevice, h->stream));
    // bank-conflict-free exchange layout of the pipelined ingest kernel (vectors of up to 48 registers per lane: beyond that the kernel has no registers for the offsets)
    h->exchange_ready = false;
    ExchangeLayoutHost ex;
    if (dim % 32 == 0 && dim / 32 <= 48 && build_exchange_layout(int(dim), h->rot.packed[1].data(), ex)) {
        TV_CUDA(h->d_store_bank.reserve(dim));
        TV_CUDA(h->d_perm1_exchange.reserve(dim));
        TV_CUDA(cudaMemcpyAsync(h->d_store_bank.ptr, ex.store_bank.data(), dim, cudaMemcpyHostToDevice, h->stream));
        TV_CUDA(cudaMemcpyAsync(h->d_perm1_exchange.ptr, ex.perm1_exchange.data(), size_t(dim) * 2, cudaMemcpyHostToDevice, h->stream));
        TV_CUDA(cudaStreamSynchronize(h->stream));     // `ex` goes out of scope
        h->exchange_ready = true;
    }
    int rc = upload_codebook(h);
    if (rc != TV_OK) return rc;
    h->tables_ready = true;
    return TV_OK;
}

int upload_calibration(tv_index *h) {
    if (h->shift.empty()) return TV_OK;
    const size_t dim = h->dim;
    std::vector<float> buf(3 * dim);
    for (size_t d = 0; d < dim; ++d) {
        buf[d] = h->shift[d];
        buf[dim + d] = h->scale_tq[d];
        buf[2 * dim + d] = 1.0f / h->scale_tq[d];     // encode.rs:593
    }
    TV_CUDA(h->d_calib.reserve(3 * dim));
    TV_CUDA(cudaMemcpyAsync(h->d_calib.ptr, buf.data(), buf.size() * 4, cudaMemcpyHostToDevice, h->stream));
    TV_CUDA(cudaStreamSynchronize(h->stream));
    return TV_OK;
}

// Grows the code / scale arrays to hold `n_total` vectors.  New space is zero so that padding lanes read
// as zero bytes (pack.rs:347-358).  Growth is geometric (x1.5) and copies once.
int ensure_capacity(tv_index *h, size_t n_total) {
    TV_CUDA(injected_failure(h));
    const size_t blocks = (n_total + kBlock - 1) / kBlock;
    const size_t block_bytes = size_t(h->ngroups) * kBlock;
    if (blocks > h->code_blocks_cap) {
        size_t new_cap = std::max(blocks, h->code_blocks_cap + h->code_blocks_cap / 2);
        new_cap = std::max<size_t>(new_cap, 64);
        uint8_t *fresh = nullptr;
        cudaError_t e = cudaMalloc(&fresh, new_cap * block_bytes);
        if (e != cudaSuccess && new_cap > blocks) {      // retry with the exact size before giving up
            cudaGetLastError();
            new_cap = blocks;
            e = cudaMalloc(&fresh, new_cap * block_bytes);
        }
        TV_CUDA(e);
        const size_t used = ((h->n + kBlock - 1) / kBlock) * block_bytes;
        if (used) TV_CUDA(cudaMemcpyAsync(fresh, h->d_codes, used, cudaMemcpyDeviceToDevice, h->stream));
        TV_CUDA(cudaMemsetAsync(fresh + used, 0, new_cap * block_bytes - used, h->stream));
        TV_CUDA(cudaStreamSynchronize(h->stream));
        if (h->d_codes) cudaFree(h->d_codes);
        h->d_codes = fresh;
        h->code_blocks_cap = new_cap;
        h->expanded.drop();                    // sized by the capacity: rebuilt by the next search that wants it
    }
    if (n_total > h->scales_cap) {
        size_t new_cap = std::max(n_total, h->scales_cap + h->scales_cap / 2);
        new_cap = std::max<size_t>(new_cap, 2048);
        float *fresh = nullptr;
        TV_CUDA(cudaMalloc(&fresh, new_cap * sizeof(float)));
        if (h->n) TV_CUDA(cudaMemcpyAsync(fresh, h->d_scales, h->n * sizeof(float), cudaMemcpyDeviceToDevice, h->stream));
        TV_CUDA(cudaStreamSynchronize(h->stream));
        if (h->d_scales) cudaFree(h->d_scales);
        h->d_scales = fresh;
        h->scales_cap = new_cap;
    }
    return TV_OK;
}

__global__ void clear_slots_kernel(uint8_t *codes, int ng, int64_t slot_begin, int64_t slot_end) {
    // zeroes the code bytes of slots [slot_begin, slot_end)
    const int64_t total = (slot_end - slot_begin) * ng;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
        const int64_t slot = slot_begin + i / ng;
        const int g = int(i % ng);
        codes[((slot / 32) * ng + g) * 32 + (slot % 32)] = 0;
    }
}

// swap_remove on the blocked array: pack::move_lane + pack::zero_lane (pack.rs:174-246).
__global__ void move_lane_kernel(uint8_t *codes, float *scales, int ng, int64_t src, int64_t dst) {
    for (int g = blockIdx.x * blockDim.x + threadIdx.x; g < ng; g += gridDim.x * blockDim.x) {
        uint8_t *s = codes + ((src / 32) * ng + g) * 32 + (src % 32);
        if (src != dst) codes[((dst / 32) * ng + g) * 32 + (dst % 32)] = *s;
        *s = 0;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0 && src != dst) scales[dst] = scales[src];
}

// One row's byte-groups <-> a contiguous buffer (pack::read_code / write_code over a lane, pack.rs:1113-1160).
__global__ void gather_row_kernel(const uint8_t *codes, int ng, int64_t slot, uint8_t *out) {
    for (int g = blockIdx.x * blockDim.x + threadIdx.x; g < ng; g += gridDim.x * blockDim.x)
        out[g] = codes[((slot / 32) * ng + g) * 32 + (slot % 32)];
}
__global__ void scatter_row_kernel(uint8_t *codes, int ng, int64_t slot, const uint8_t *in) {
    for (int g = blockIdx.x * blockDim.x + threadIdx.x; g < ng; g += gridDim.x * blockDim.x)
        codes[((slot / 32) * ng + g) * 32 + (slot % 32)] = in[g];
}

int validate_dim_for_add(tv_index *h, size_t dim) {
    // add_2d, lib.rs:1114-1133
    if (h->dim != 0) {
        if (h->dim != dim)
            return fail(h, TV_ERR_DIM_MISMATCH, "dimension mismatch: index has dim " + std::to_string(h->dim) + ", got " + std::to_string(dim));
        return TV_OK;
    }
    if (dim == 0) return fail(h, TV_ERR_ZERO_DIM, "dim must be non-zero");
    if (dim % 8 != 0) return fail(h, TV_ERR_DIM_NOT_MULTIPLE_OF_8, "dim " + std::to_string(dim) + " is not a multiple of 8");
    if (dim > size_t(kMaxDim)) return fail(h, TV_ERR_DIM_TOO_LARGE, "dim " + std::to_string(dim) + " exceeds " + std::to_string(kMaxDim));
    return TV_OK;
}

// Encodes n rows (host or device memory) onto the end of the index.  All-or-nothing.
int add_rows(tv_index *h, const float *x, size_t n, size_t dim, bool on_device) {
    int rc = validate_dim_for_add(h, dim);
    if (rc != TV_OK) return rc;
    if (n == 0) return TV_OK;
    if (h->n + n > 0xfffffff0ull) return fail(h, TV_ERR_UNSUPPORTED, "more than 2^32 - 16 vectors per device shard");
    TV_CUDA(cudaSetDevice(h->device));
    const bool was_lazy = h->dim == 0;
    if (was_lazy) h->dim = dim;
    rc = ensure_tables(h);
    if (rc == TV_OK) rc = ensure_capacity(h, h->n + n);
    if (rc != TV_OK) {
        if (was_lazy) { h->dim = 0; h->tables_ready = false; }
        return rc;
    }
    const int V = ingest_vectors_per_pass(int(dim), h->ngroups, h->smem_limit);
    if (V == 0) return fail(h, TV_ERR_UNSUPPORTED, "dim too large for the ingest kernel's shared memory");

    h->h_flags->first_invalid = ~0ull;
    h->h_flags->error = 0;
    TV_CUDA(cudaMemcpyAsync(&h->d_flags->first_invalid, &h->h_flags->first_invalid, 8, cudaMemcpyHostToDevice, h->stream));
    TV_CUDA(cudaMemcpyAsync(&h->d_flags->error, &h->h_flags->error, 4, cudaMemcpyHostToDevice, h->stream));

    IngestParams p{};
    p.dim = int(dim); p.bits = h->bits; p.ngroups = h->ngroups;
    p.perm0 = h->d_perm.ptr; p.perm1 = h->d_perm.ptr + dim;
    p.inv_sqrt_block = h->rot.inv_sqrt_block;
    p.boundaries = h->d_codebook.ptr; p.centroids = h->d_codebook.ptr + 16;
    if (!h->shift.empty()) { p.shift = h->d_calib.ptr; p.scale_tq = h->d_calib.ptr + dim; p.inv_scale_tq = h->d_calib.ptr + 2 * dim; }
    p.codes = h->d_codes; p.scales = h->d_scales;
    p.first_invalid = &h->d_flags->first_invalid;

    // Device input is encoded in place.  Host input goes through pinned staging in chunks of about 64 MB,
    // double buffered: host threads copy chunk i+1 into pinned memory while chunk i crosses the bus on the copy
    // stream and chunk i-1 is encoded on the handle's stream.
    const size_t chunk_rows = on_device ? n : std::max<size_t>(1, std::min<size_t>(n, (size_t(64) << 20) / (dim * 4)));
    if (!on_device) {
        if (!h->copy_stream) {
            TV_CUDA(cudaStreamCreateWithFlags(&h->copy_stream, cudaStreamNonBlocking));
            for (int b = 0; b < 2; ++b) {
                TV_CUDA(cudaEventCreateWithFlags(&h->ev_copied[b], cudaEventDisableTiming));
                TV_CUDA(cudaEventCreateWithFlags(&h->ev_consumed[b], cudaEventDisableTiming));
            }
        }
        for (int b = 0; b < 2; ++b) {
            TV_CUDA(h->h_add[b].reserve(chunk_rows * dim));
            TV_CUDA(h->d_add[b].reserve(chunk_rows * dim));
        }
    }
    const size_t copy_threads = std::min<size_t>(16, std::max(1u, std::thread::hardware_concurrency()));
    // page-locked input (cudaHostAlloc / cudaHostRegister) is read by the copy engine directly
    bool src_pinned = false;
    if (!on_device) {
        cudaPointerAttributes attr{};
        if (cudaPointerGetAttributes(&attr, x) == cudaSuccess) src_pinned = attr.type == cudaMemoryTypeHost;
        else cudaGetLastError();
    }
    // A failure after the first launch leaves bytes in lanes past `len`: they are cleared again before the
    // call returns, so that a failed add leaves the index exactly as it was (lib.rs:889-930).
    cudaError_t step_err = cudaSuccess;
    const char *step_what = "";
#define TV_STEP(expr)                                              \
    {                                                              \
        step_err = (expr);                                         \
        if (step_err != cudaSuccess) { step_what = #expr; break; } \
    }
    TV_CUDA(cudaEventRecord(h->ev0, h->stream));
    size_t chunk_index = 0;
    for (size_t done = 0; done < n; done += chunk_rows, ++chunk_index) {
        const size_t rows = std::min(chunk_rows, n - done);
        const float *src = x + done * dim;
        TV_STEP(injected_failure(h));
        if (!on_device) {
            const int b = int(chunk_index & 1);
            if (chunk_index >= 2) TV_STEP(cudaEventSynchronize(h->ev_consumed[b]));   // the encode of chunk i-2 has read d_add[b]
            const size_t bytes = rows * dim * 4;
            const float *h_src = h->h_add[b].ptr;
            if (src_pinned) {
                h_src = src;
            } else if (bytes < (size_t(4) << 20) || copy_threads == 1) {
                std::memcpy(h->h_add[b].ptr, src, bytes);
            } else {
                std::vector<std::thread> pool;
                for (size_t t = 0; t < copy_threads; ++t) {
                    const size_t lo = bytes * t / copy_threads / 64 * 64, hi = t + 1 == copy_threads ? bytes : bytes * (t + 1) / copy_threads / 64 * 64;
                    pool.emplace_back([=] { std::memcpy(reinterpret_cast<char *>(h->h_add[b].ptr) + lo, reinterpret_cast<const char *>(src) + lo, hi - lo); });
                }
                for (auto &th : pool) th.join();
            }
            TV_STEP(cudaMemcpyAsync(h->d_add[b].ptr, h_src, bytes, cudaMemcpyHostToDevice, h->copy_stream));
            TV_STEP(cudaEventRecord(h->ev_copied[b], h->copy_stream));
            TV_STEP(cudaStreamWaitEvent(h->stream, h->ev_copied[b], 0));
            src = h->d_add[b].ptr;
        }
        p.x = src; p.n = int64_t(rows); p.slot0 = int64_t(h->n + done); p.row_base = int64_t(done);
        // rows that complete a partly filled block go through the block-at-a-time kernel, whole blocks
        // through the pipelined one where it applies
        int64_t head = rows;
        if (h->ingest_pipeline && h->qgrid.cells != nullptr &&
            ingest_fast_supported(int(dim), h->bits, h->ngroups, p.shift != nullptr, src, h->smem_limit))
            head = std::min<int64_t>(int64_t(rows), (kBlockLanes - p.slot0 % kBlockLanes) % kBlockLanes);
        if (head > 0) {
            p.n = head;
            mark_begin(h);
            TV_STEP(launch_ingest(p, V, h->stream));
            mark_end(h);
            h->launches++;
        }
        if (int64_t(rows) > head) {
            p.x = src + head * int64_t(dim); p.n = int64_t(rows) - head; p.slot0 += head; p.row_base += head;
            p.exact_sums = h->ingest_pipeline == 2;
            if (h->exchange_ready) { p.store_bank = h->d_store_bank.ptr; p.perm1_exchange = h->d_perm1_exchange.ptr; }
            mark_begin(h);
            TV_STEP(launch_ingest_fast(p, h->qgrid, h->sm_count, h->smem_limit, &h->d_flags->error, h->stream));
            mark_end(h);
            h->launches++;
        }
        if (!on_device) TV_STEP(cudaEventRecord(h->ev_consumed[chunk_index & 1], h->stream));
    }
#undef TV_STEP
    if (step_err != cudaSuccess) {
        cudaGetLastError();
        cudaStreamSynchronize(h->stream);
        if (h->copy_stream) cudaStreamSynchronize(h->copy_stream);
        const int64_t total = int64_t(n) * h->ngroups;
        clear_slots_kernel<<<unsigned(std::min<int64_t>((total + 255) / 256, 65535)), 256, 0, h->stream>>>(
            h->d_codes, h->ngroups, int64_t(h->n), int64_t(h->n + n));
        cudaStreamSynchronize(h->stream);
        h->marks.used = 0;
        if (was_lazy) { h->dim = 0; h->tables_ready = false; }
        return fail(h, step_err == cudaErrorMemoryAllocation ? TV_ERR_OUT_OF_MEMORY : TV_ERR_CUDA,
                    std::string(step_what) + ": " + cudaGetErrorString(step_err));
    }
    TV_CUDA(cudaEventRecord(h->ev1, h->stream));
    TV_CUDA(cudaMemcpyAsync(&h->h_flags->first_invalid, &h->d_flags->first_invalid, 8, cudaMemcpyDeviceToHost, h->stream));
    TV_CUDA(cudaMemcpyAsync(&h->h_flags->error, &h->d_flags->error, 4, cudaMemcpyDeviceToHost, h->stream));
    TV_CUDA(cudaStreamSynchronize(h->stream));
    cudaEventElapsedTime(&h->last_ms, h->ev0, h->ev1);
    collect_marks(h);
    if (h->h_flags->error != 0) {
        if (was_lazy) { h->dim = 0; h->tables_ready = false; }
        return fail(h, TV_ERR_DEVICE_TIMEOUT, "the ingest kernel gave up waiting for a staged row (code " + std::to_string(h->h_flags->error) + ")");
    }
    if (h->h_flags->first_invalid != ~0ull) {
        // roll back: the new lanes must read as zero again, nothing else was touched
        const int64_t total = int64_t(n) * h->ngroups;
        clear_slots_kernel<<<unsigned(std::min<int64_t>((total + 255) / 256, 65535)), 256, 0, h->stream>>>(
            h->d_codes, h->ngroups, int64_t(h->n), int64_t(h->n + n));
        cudaStreamSynchronize(h->stream);
        const unsigned long long flat = h->h_flags->first_invalid;
        h->err_vec = size_t(flat / dim); h->err_coord = size_t(flat % dim);
        if (on_device) cudaMemcpy(&h->err_value, x + flat, 4, cudaMemcpyDeviceToHost);
        else h->err_value = x[flat];
        if (was_lazy) { h->dim = 0; h->tables_ready = false; }
        return fail(h, TV_ERR_INVALID_INPUT_VALUE,
                    "vector " + std::to_string(h->err_vec) + " coordinate " + std::to_string(h->err_coord) +
                        " is not finite or exceeds 1e16 in magnitude (value " + std::to_string(h->err_value) + ")");
    }
    h->n += n;
    mutation_done(h);
    return TV_OK;
}

struct MaskSpec {
    const uint8_t *bool_host = nullptr; size_t bool_len = 0;
    const uint64_t *words_host = nullptr; size_t n_words = 0;
    const uint64_t *words_device = nullptr;
    const uint32_t *slots_host = nullptr; size_t n_slots = 0;
    const uint64_t *ids_host = nullptr; size_t n_ids = 0;   // allowlist ids, resolved by the device table
    bool prepared = false;                 // use the handle's prepared mask
    bool any() const { return bool_host || words_host || words_device || slots_host || ids_host || prepared; }
};

int candidate_capacity(size_t k) { return k <= 512 ? 4096 : 8192; }
constexpr size_t kPageK = 4096;            // most results one selection pass keeps per query; larger k runs in pages

// Takes a search context from the handle's pool for the duration of a call.
struct CtxLease {
    tv_index *h;
    SearchCtx *c = nullptr;
    explicit CtxLease(tv_index *handle) : h(handle) {
        std::unique_lock<std::mutex> g(h->ctx_mu);
        for (;;) {
            for (int i = 0; i < kSearchCtxs; ++i)
                if (!h->ctx[i].busy) { c = &h->ctx[i]; break; }
            if (c) break;
            h->ctx_cv.wait(g);
        }
        c->busy = true;
    }
    ~CtxLease() {
        { std::lock_guard<std::mutex> g(h->ctx_mu); c->busy = false; }
        h->ctx_cv.notify_one();
    }
};

// The device buffers one search runs on: the context's arrays, or the fixed array of the allocation-free entry point.
struct SearchScratch {
    float *q_rot, *qscale, *qbias;
    int8_t *weights;
    uint32_t *wfrag;
    uint8_t *luts;
    uint64_t *cand, *thr, *topk, *lo;      // lo: lowest admissible key per query (paged top-k), or nullptr
    uint32_t *cnt;
    size_t w_rows, dim_pad, lut_pitch;
    int cap;
    bool allow_tc;
};

struct MaskOnDevice {
    const uint64_t *words = nullptr;
    const uint32_t *live = nullptr;
    const uint32_t *n_live = nullptr;
    const unsigned long long *n_allowed = nullptr;
};

// Brings the device id table up to date on stream `st` (a rebuild from slot_to_id, or the changes since the last time)
// and makes `st` wait for whatever update last touched it.
int idtab_sync(tv_index *h, cudaStream_t st) {
    DeviceIdTable &t = h->idtab;
    std::lock_guard<std::mutex> g(t.mu);
    if (!t.ev) TV_CUDA(cudaEventCreateWithFlags(&t.ev, cudaEventDisableTiming));
    const size_t n = h->slot_to_id.size();
    const size_t cap = t.log2cap ? size_t(1) << t.log2cap : 0;
    if (!t.valid || (t.used + t.pending.size()) * 10 > cap * 7) {
        int lg = 16;
        while ((size_t(1) << lg) < 2 * n) ++lg;
        TV_CUDA(injected_failure(h));
        TV_CUDA(t.keys.reserve(size_t(1) << lg));
        TV_CUDA(t.vals.reserve(size_t(1) << lg));
        TV_CUDA(t.d_ids.reserve(n));
        t.log2cap = lg;
        TV_CUDA(cudaMemsetAsync(t.keys.ptr, 0xff, (size_t(1) << lg) * 8, st));
        TV_CUDA(cudaMemcpyAsync(t.d_ids.ptr, h->slot_to_id.data(), n * 8, cudaMemcpyHostToDevice, st));
        TV_CUDA(launch_idtab_insert(t.keys.ptr, t.vals.ptr, lg, t.d_ids.ptr, int64_t(n), 0, st));
        h->launches++;
        t.used = n; t.valid = true; t.pending.clear();
    } else if (!t.pending.empty()) {
        // the last operation on an id wins; the kernel wants every id once
        std::unordered_map<uint64_t, uint32_t> last;
        last.reserve(t.pending.size() * 2);
        for (const auto &op : t.pending) last[op.first] = op.second;
        std::vector<uint64_t> ids;
        std::vector<uint32_t> slots;
        ids.reserve(last.size()); slots.reserve(last.size());
        for (const auto &kv : last) { ids.push_back(kv.first); slots.push_back(kv.second); }
        TV_CUDA(t.d_ids.reserve(ids.size()));
        TV_CUDA(t.d_slots.reserve(ids.size()));
        TV_CUDA(cudaMemcpyAsync(t.d_ids.ptr, ids.data(), ids.size() * 8, cudaMemcpyHostToDevice, st));
        TV_CUDA(cudaMemcpyAsync(t.d_slots.ptr, slots.data(), slots.size() * 4, cudaMemcpyHostToDevice, st));
        TV_CUDA(launch_idtab_upsert(t.keys.ptr, t.vals.ptr, t.log2cap, t.d_ids.ptr, t.d_slots.ptr, int64_t(ids.size()), st));
        TV_CUDA(cudaStreamSynchronize(st));          // the host vectors above are pageable: keep them until the copies are done
        h->launches++;
        t.used += ids.size();
        t.pending.clear();
    } else {
        TV_CUDA(cudaStreamWaitEvent(st, t.ev, 0));
        return TV_OK;
    }
    TV_CUDA(cudaEventRecord(t.ev, st));
    return TV_OK;
}

// Uploads / packs the allow-mask of a call and compacts its live blocks.  `words_buf` / `live_buf` receive the data,
// the two counters are zeroed by the caller.
int build_mask(tv_index *h, cudaStream_t st, const MaskSpec &mask, DeviceArray<uint64_t> &words_buf,
               DeviceArray<uint8_t> &bool_buf, DeviceArray<uint32_t> &slots_buf, DeviceArray<uint32_t> &live_buf,
               DeviceArray<uint64_t> &ids_buf, unsigned long long *d_first_unknown,
               unsigned long long *d_n_allowed, uint32_t *d_n_live, MaskOnDevice &out) {
    const size_t n = h->n, n_words = (n + 63) / 64, n_blocks = (n + kBlock - 1) / kBlock;
    TV_CUDA(injected_failure(h));
    TV_CUDA(words_buf.reserve(n_words));
    if (mask.words_device) {
        TV_CUDA(cudaMemcpyAsync(words_buf.ptr, mask.words_device, n_words * 8, cudaMemcpyDeviceToDevice, st));
    } else if (mask.words_host) {
        TV_CUDA(cudaMemcpyAsync(words_buf.ptr, mask.words_host, n_words * 8, cudaMemcpyHostToDevice, st));
    } else if (mask.ids_host) {
        // the allowlist itself goes to the device; the id table there turns it into mask bits (id_map.rs:670-683)
        TV_CUDA(ids_buf.reserve(mask.n_ids));
        TV_CUDA(cudaMemsetAsync(words_buf.ptr, 0, n_words * 8, st));
        TV_CUDA(cudaMemcpyAsync(ids_buf.ptr, mask.ids_host, mask.n_ids * 8, cudaMemcpyHostToDevice, st));
        int rc = idtab_sync(h, st);
        if (rc != TV_OK) return rc;
        TV_CUDA(launch_idtab_lookup(h->idtab.keys.ptr, h->idtab.vals.ptr, h->idtab.log2cap, ids_buf.ptr, int64_t(mask.n_ids), words_buf.ptr,
                                    d_first_unknown, st));
        h->launches++;
    } else if (mask.bool_host) {
        TV_CUDA(bool_buf.reserve(n));
        TV_CUDA(cudaMemcpyAsync(bool_buf.ptr, mask.bool_host, n, cudaMemcpyHostToDevice, st));
        TV_CUDA(launch_pack_bool_mask(bool_buf.ptr, int64_t(n), words_buf.ptr, st));
        h->launches++;
    } else {
        TV_CUDA(slots_buf.reserve(mask.n_slots));
        TV_CUDA(cudaMemsetAsync(words_buf.ptr, 0, n_words * 8, st));
        TV_CUDA(cudaMemcpyAsync(slots_buf.ptr, mask.slots_host, mask.n_slots * 4, cudaMemcpyHostToDevice, st));
        TV_CUDA(launch_scatter_slots(slots_buf.ptr, int64_t(mask.n_slots), words_buf.ptr, st));
        h->launches++;
    }
    TV_CUDA(live_buf.reserve(n_blocks));
    TV_CUDA(launch_mask_stats(words_buf.ptr, int64_t(n), d_n_allowed, live_buf.ptr, d_n_live, st));
    h->launches++;
    out.words = words_buf.ptr; out.live = live_buf.ptr; out.n_live = d_n_live; out.n_allowed = d_n_allowed;
    return TV_OK;
}

ScanParams base_scan_params(const tv_index *h, int mode) {
    ScanParams sp{};
    sp.codes = h->d_codes; sp.vec_scales = h->d_scales; sp.n = int64_t(h->n); sp.ngroups = h->ngroups; sp.bits = h->bits;
    sp.mode = mode;
    for (int w = 0; w < 4; ++w) {
        uint32_t word = 0;
        for (int b = 0; b < 4; ++b) word |= uint32_t(uint8_t(h->levels[4 * w + b])) << (8 * b);
        sp.level_words[w] = word;
    }
    sp.pd_split = h->pd_split;
    return sp;
}

// Which kernel family a batch runs on.
struct ScanPlan {
    bool use_tc = false;       // tensor-memory scan (tcgen05)
    bool use_small = false;    // scan_small_kernel (up to 16 permute-dot queries)
    int lut_width = 0;         // queries per launch of the CUDA-core LUT scan
};

int plan_scan(tv_index *h, int mode, size_t nq, bool allow_tc, ScanPlan &plan) {
    const int ng = h->ngroups;
    // measured on 1.25 M and 10 M x 1536 4-bit: mma.sync 0.67 / 3.6 ms up to 32 queries, 0.89 / 5.1 ms from 33 on,
    // tcgen05 0.83 / 5.1 ms flat; on 1 M x 3072 2-bit the CUDA-core LUT scan costs 0.5 ms per query beyond 4,
    // tcgen05 4.2 ms flat
    // with the int8 copy of the index the tensor-memory scan is bound by reading it (2.85 ms at 33 queries on 10 M x 1536)
    // and beats the mma.sync scan of 17 - 32 queries (3.1 ms); without the copy it expands codes and does not (4.7 ms)
    bool copy_expected = false;
    if (mode == TV_SCORE_PERMUTE_DOT && h->tc_expanded != 0) {
        std::lock_guard<std::mutex> g(h->expanded.mu);
        copy_expected = h->tc_expanded == 2 || h->expanded.refused_at_cap != h->code_blocks_cap * kBlock;
    }
    const int64_t tc_from = h->mma_min_batch >= 0 ? h->mma_min_batch : (mode == TV_SCORE_PERMUTE_DOT ? (copy_expected ? 17 : 33) : 8);
    plan.use_tc = allow_tc && tc_from > 0 && int64_t(nq) >= tc_from && scan_tc_supported(h->bits, mode, ng);
    if (mode != TV_SCORE_PERMUTE_DOT) {
        plan.lut_width = scan_lut_width(ng, h->smem_limit);
        if (!plan.use_tc && plan.lut_width == 0) {
            // not even one query's tables fit in shared memory: the tensor-memory scan takes the tables from global memory
            if (allow_tc && scan_tc_supported(h->bits, mode, ng)) plan.use_tc = true;
            else return fail(h, TV_ERR_UNSUPPORTED, "the u8 tables of one query (" + std::to_string(size_t(ng) * 32) +
                                                        " bytes) exceed shared memory and this score mode has no tensor-memory scan");
        }
    }
    return TV_OK;
}

// Brings the int8 copy of the index (scan_tc_dense.cu) up to date on `st`: allocates it when policy and free memory
// allow, expands the rows appended and the blocks changed in place since the last time.  *usable = false when there
// is no copy to scan (switched off, or no room); the caller then scans the codes.
int expanded_sync(tv_index *h, cudaStream_t st, const uint32_t level_words[4], bool *usable) {
    *usable = false;
    ExpandedCopy &x = h->expanded;
    if (h->tc_expanded == 0 || h->n == 0) return TV_OK;
    std::lock_guard<std::mutex> g(x.mu);
    if (!x.ev) TV_CUDA(cudaEventCreateWithFlags(&x.ev, cudaEventDisableTiming));
    const size_t rows = h->code_blocks_cap * kBlock;
    const int pitch = expanded_pitch(int(h->dim));
    if (x.rows_cap != rows || x.pitch != pitch || !x.levels.ptr) {
        if (x.refused_at_cap == rows && h->tc_expanded != 2) return TV_OK;
        const size_t bytes = rows * size_t(pitch);
        size_t free_b = 0, total_b = 0;
        TV_CUDA(cudaMemGetInfo(&free_b, &total_b));
        // keep a tenth of the device (at least 1 GiB) free for scratch and for the growth of the index
        const size_t keep = std::max<size_t>(total_b / 10, size_t(1) << 30);
        x.drop();
        cudaError_t e = cudaErrorMemoryAllocation;
        if (h->tc_expanded == 2 || free_b >= bytes + keep) e = x.levels.reserve(bytes);
        if (e != cudaSuccess) {
            cudaGetLastError();
            x.refused_at_cap = rows;
            if (h->tc_expanded == 2) return fail(h, TV_ERR_CUDA, "no room for the int8 copy of the index (" + std::to_string(bytes) + " bytes)");
            return TV_OK;
        }
        // padding columns and rows are never cleared: padding columns meet zero query weights, padding rows are not read out
        x.rows_cap = rows; x.pitch = pitch;
    }
    bool work = false;
    if (!x.dirty.empty()) {
        TV_CUDA(x.d_dirty.reserve(x.dirty.size()));
        TV_CUDA(cudaMemcpyAsync(x.d_dirty.ptr, x.dirty.data(), x.dirty.size() * 4, cudaMemcpyHostToDevice, st));   // pageable: staged before the call returns
        TV_CUDA(launch_expand_blocks(h->d_codes, h->ngroups, x.d_dirty.ptr, 0, uint32_t(x.dirty.size()), x.levels.ptr, pitch, level_words,
                                     h->sm_count, st));
        h->launches++;
        x.dirty.clear();
        work = true;
    }
    if (x.rows_valid < h->n) {
        const size_t first = x.rows_valid / kBlock, end = (h->n + kBlock - 1) / kBlock;
        TV_CUDA(launch_expand_blocks(h->d_codes, h->ngroups, nullptr, uint32_t(first), uint32_t(end - first), x.levels.ptr, pitch, level_words,
                                     h->sm_count, st));
        h->launches++;
        x.rows_valid = h->n;
        work = true;
    }
    if (work) TV_CUDA(cudaEventRecord(x.ev, st));
    else TV_CUDA(cudaStreamWaitEvent(st, x.ev, 0));
    *usable = true;
    return TV_OK;
}

// Query preparation, then scan + select over a geometric chunk schedule, all enqueued on `st`.
//   careful: chunks never exceed the candidate capacity, so no list can overflow whatever the data order.
int enqueue_search(tv_index *h, cudaStream_t st, Marks *marks, const SearchScratch &S, const ScanPlan &plan, int mode,
                   size_t nq, size_t kk, const MaskOnDevice &m, uint32_t *d_overflow, uint32_t *d_error, bool careful) {
    const size_t n = h->n;
    const int ng = h->ngroups;
    const size_t n_blocks = (n + kBlock - 1) / kBlock;
    const int mt_total = int((nq + 15) / 16);
    CandidateBuffers cb{};
    cb.cand = S.cand; cb.cnt = S.cnt; cb.thr = S.thr; cb.topk = S.topk; cb.lo = S.lo;
    cb.overflow = d_overflow; cb.error = d_error; cb.cap = S.cap; cb.k = int(kk);

    ScanParams sp = base_scan_params(h, mode);
    sp.qscale = S.qscale; sp.qbias = S.qbias;
    sp.mask = m.words; sp.live_blocks = m.live; sp.n_live = m.n_live;
    sp.cb = cb; sp.wfrag = S.wfrag; sp.mtiles_total = mt_total; sp.luts = S.luts; sp.lut_pitch = int(S.lut_pitch);
    const bool use_small = plan.use_small && !plan.use_tc;
    bool use_dense = false;
    if (plan.use_tc && scan_tc_dense_supported(h->bits, mode, ng) && int(S.dim_pad) == expanded_pitch(int(h->dim))) {
        int rc = expanded_sync(h, st, sp.level_words, &use_dense);
        if (rc != TV_OK) return rc;
    }

    TV_CUDA(cudaMemsetAsync(S.cnt, 0, nq * 4, st));
    TV_CUDA(cudaMemsetAsync(S.thr, 0xff, nq * 8, st));
    TV_CUDA(cudaMemsetAsync(S.topk, 0xff, nq * kk * 8, st));
    // Chunk 0 holds at most `cap` vectors, so every one of them may pass.  Later chunks grow so that the
    // expected number of candidates per query, k * |chunk| / |seen|, stays near cap / 4.
    // The tensor-memory scan pays for dense candidates (its epilogue re-reads a 32 x 32 tile of scores
    // whenever one of them passes), so its first three chunks grow x6 each (measured against x24, x10 and others on
    // 10 M and 1.25 M vectors), then by the list-capacity rule.
    const size_t first = size_t(S.cap) / kBlock;
    const double growth = std::max(0.5, double(S.cap) / (4.0 * double(kk)));
    size_t begin = 0;
    int stage = 0;
    while (begin < n_blocks) {
        size_t len = first;
        if (!careful && begin > 0) {
            double g = growth;
            if (plan.use_tc && stage <= 3) g = std::min(g, 6.0);
            len = std::max<size_t>(first, size_t(double(begin) * g));
            if (begin + len + len / 2 >= n_blocks) len = n_blocks - begin;   // no short tail chunk
        }
        const size_t end = std::min(n_blocks, begin + len);
        sp.pos_begin = uint32_t(begin); sp.pos_end = uint32_t(end);
        // first chunk on the tensor-memory path without a filter (the host then knows how many vectors
        // the chunk holds): every key is written in place, nothing is counted
        const bool dense = plan.use_tc && stage == 0 && !careful && m.words == nullptr && S.lo == nullptr;
        sp.dense = dense ? 1 : 0;
        ++stage;
        if (plan.use_tc) {
            sp.q_base = 0; sp.nq = int(nq); sp.mtile_base = 0;
            if (marks) marks->begin(st);
            const bool wide = h->tc_wide && scan_tc_wide_supported(h->bits, mode, ng, int(nq));
            if (use_dense && h->dense_pair)
                TV_CUDA(launch_scan_tc_dense_pair(sp, h->expanded.levels.ptr, h->expanded.rows_cap, S.weights, int(S.w_rows), int(S.dim_pad),
                                                  h->sm_count, st));
            else if (use_dense)
                TV_CUDA(launch_scan_tc_dense(sp, h->expanded.levels.ptr, h->expanded.rows_cap, S.weights, int(S.w_rows), int(S.dim_pad),
                                             h->sm_count, st));
            else if (wide && mode == TV_SCORE_PERMUTE_DOT)
                TV_CUDA(launch_scan_tc_wide(sp, S.weights, int(S.w_rows), int(S.dim_pad), h->sm_count, st));
            else if (wide)
                TV_CUDA(launch_scan_tc_wide(sp, reinterpret_cast<const int8_t *>(S.luts), int(S.w_rows), int(S.lut_pitch), h->sm_count, st));
            else if (mode == TV_SCORE_PERMUTE_DOT)
                TV_CUDA(launch_scan_tc(sp, S.weights, int(S.w_rows), int(S.dim_pad), h->sm_count, h->tc_tiles, st));
            else
                TV_CUDA(launch_scan_tc(sp, reinterpret_cast<const int8_t *>(S.luts), int(S.w_rows), int(S.lut_pitch), h->sm_count, 1, st));
            if (marks) marks->end(st);
            h->launches++;
        } else if (use_small) {
            sp.q_base = 0; sp.nq = int(nq); sp.mtile_base = 0;
            if (marks) marks->begin(st);
            TV_CUDA(launch_scan_small(sp, S.weights, int(S.dim_pad), h->code_blocks_cap * size_t(ng) * kBlock, h->small_scan,
                                      h->sm_count, h->smem_limit, st));
            if (marks) marks->end(st);
            h->launches++;
        } else if (mode == TV_SCORE_PERMUTE_DOT) {
            for (size_t q0 = 0; q0 < nq; q0 += 64) {
                sp.q_base = int(q0); sp.nq = int(std::min<size_t>(64, nq - q0)); sp.mtile_base = int(q0 / 16);
                if (marks) marks->begin(st);
                TV_CUDA(launch_scan_pd(sp, h->sm_count, st));
                if (marks) marks->end(st);
                h->launches++;
            }
        } else {
            for (size_t q0 = 0; q0 < nq; q0 += size_t(plan.lut_width)) {
                sp.q_base = int(q0); sp.nq = int(std::min<size_t>(size_t(plan.lut_width), nq - q0));
                if (marks) marks->begin(st);
                TV_CUDA(launch_scan_lut(sp, h->sm_count, st));
                if (marks) marks->end(st);
                h->launches++;
            }
        }
        TV_CUDA(launch_select(cb, int(nq), dense ? int((end - sp.pos_begin) * kBlock) : 0, st));
        h->launches++;
        begin = end;
    }
    return TV_OK;
}

int enqueue_query_prep(tv_index *h, cudaStream_t st, const SearchScratch &S, const ScanPlan &plan, int mode, const float *dq,
                       size_t nq, unsigned long long *d_first_invalid) {
    const size_t dim = h->dim;
    const int ng = h->ngroups;
    const int ksteps = (ng + 15) / 16;
    const int mt_total = int((nq + 15) / 16);
    QueryPrepParams qp{};
    qp.queries = dq; qp.nq = int(nq); qp.dim = int(dim); qp.bits = h->bits; qp.ngroups = ng;
    qp.mode = mode;
    qp.perm0 = h->d_perm.ptr; qp.perm1 = h->d_perm.ptr + dim;
    qp.inv_sqrt_block = h->rot.inv_sqrt_block;
    qp.centroids = h->d_codebook.ptr + 16;
    if (!h->shift.empty()) { qp.shift = h->d_calib.ptr; qp.scale_tq = h->d_calib.ptr + dim; }
    qp.level_scale = h->level_scale;
    qp.q_rot = S.q_rot; qp.qscale = S.qscale; qp.qbias = S.qbias;
    qp.luts = S.luts; qp.lut_pitch = int(S.lut_pitch); qp.weights = S.weights; qp.dim_pad = int(S.dim_pad);
    qp.wfrag = S.wfrag; qp.mtiles_total = mt_total;
    qp.first_invalid = d_first_invalid;
    if (mode == TV_SCORE_PERMUTE_DOT) {
        TV_CUDA(cudaMemsetAsync(S.wfrag, 0, size_t(ksteps) * mt_total * 32 * 16, st));
        if (plan.use_tc) TV_CUDA(cudaMemsetAsync(S.weights, 0, S.w_rows * S.dim_pad, st));
    } else if (plan.use_tc) {
        TV_CUDA(cudaMemsetAsync(S.luts, 0, S.w_rows * S.lut_pitch, st));
    }
    TV_CUDA(launch_query_prep(qp, st));
    h->launches++;
    return TV_OK;
}

// Reads the status words of a finished call and turns them into an error, if any.  `queries` (host or device) is
// only used to fetch the offending value.
int check_flags(tv_index *h, const DeviceFlags *f, const float *queries, bool queries_on_device, cudaStream_t st) {
    if (f->error) return fail(h, TV_ERR_DEVICE_TIMEOUT, "a device-side wait ran out of polls");
    if (f->first_invalid != ~0ull) {
        const unsigned long long flat = f->first_invalid;
        float value = 0.f;
        if (queries_on_device) {
            cudaMemcpyAsync(&value, queries + flat, 4, cudaMemcpyDeviceToHost, st);
            cudaStreamSynchronize(st);
        } else {
            value = queries[flat];
        }
        {
            std::lock_guard<std::mutex> g(h->stat_mu);
            h->err_vec = size_t(flat / h->dim); h->err_coord = size_t(flat % h->dim); h->err_value = value;
        }
        return fail(h, TV_ERR_INVALID_QUERY_VALUE,
                    "query " + std::to_string(flat / h->dim) + " coordinate " + std::to_string(flat % h->dim) +
                        " is not finite or exceeds 1e16 in magnitude");
    }
    return TV_OK;
}

// The whole search on a context's stream.  Results land in c.d_scores / c.d_slots (row stride k) unless
// out_scores_dev is given (row stride k_eff).  The caller holds the handle's lock (shared is enough).
int search_core(tv_index *h, SearchCtx &c, const float *queries, bool queries_on_device, size_t nq, size_t k, const MaskSpec &mask,
                float *out_scores_dev, int64_t *out_slots_dev, size_t *k_eff_out, uint64_t *out_keys_dev = nullptr,
                uint64_t key_offset = 0) {
    const size_t dim = h->dim, n = h->n;
    const int ng = h->ngroups;
    const int mode = resolve_mode(h);
    const size_t kk = std::min(k, n);
    *k_eff_out = 0;
    if (nq == 0 || kk == 0) return TV_OK;
    TV_CUDA(cudaSetDevice(h->device));
    cudaStream_t st = c.stream;
    // Results beyond kPageK per query come in pages: page r keeps the kPageK best keys above the last key of page
    // r - 1 (keys are unique: they carry the slot), one full scan each.  Exact for any k <= len, slow by design.
    const size_t pages = (kk + kPageK - 1) / kPageK;
    const size_t k_page = pages == 1 ? kk : kPageK;
    const int cap = candidate_capacity(k_page);
    const size_t nq_pad = (nq + 15) / 16 * 16;
    const int mt_total = int(nq_pad / 16);
    const size_t dim_pad = (dim + 127) / 128 * 128;
    const int ksteps = (ng + 15) / 16;
    const size_t lut_pitch = size_t((ng + 3) / 4 * 4) * 32;

    ScanPlan plan;
    int rc = plan_scan(h, mode, nq, pages == 1, plan);
    if (rc != TV_OK) return rc;

    // ---- buffers ----
    TV_CUDA(injected_failure(h));
    if (!queries_on_device) TV_CUDA(c.d_stage.reserve(nq * dim));
    TV_CUDA(c.d_qrot.reserve(nq * dim));
    TV_CUDA(c.d_qscale.reserve(nq_pad));
    TV_CUDA(c.d_qbias.reserve(nq_pad));
    const size_t w_rows = (nq + 255) / 256 * 256;
    if (mode == TV_SCORE_PERMUTE_DOT) {
        TV_CUDA(c.d_weights.reserve(w_rows * dim_pad));
        TV_CUDA(c.d_wfrag.reserve(size_t(ksteps) * mt_total * 32 * 4));
    } else {
        TV_CUDA(c.d_luts.reserve(w_rows * lut_pitch));           // padded to whole query groups and whole K slabs for the tensor path
    }
    TV_CUDA(c.d_cand.reserve(nq * size_t(cap)));
    TV_CUDA(c.d_cnt.reserve(nq));
    TV_CUDA(c.d_thr.reserve(nq));
    TV_CUDA(c.d_topk.reserve(nq * k_page));
    if (pages > 1) {
        TV_CUDA(c.d_floor.reserve(nq));
        TV_CUDA(c.d_keys_all.reserve(nq * kk));
    }
    if (!out_scores_dev) {
        TV_CUDA(c.d_scores.reserve(nq * kk));
        TV_CUDA(c.d_slots.reserve(nq * kk));
    }

    SearchScratch S{};
    S.q_rot = c.d_qrot.ptr; S.qscale = c.d_qscale.ptr; S.qbias = c.d_qbias.ptr; S.weights = c.d_weights.ptr;
    S.wfrag = c.d_wfrag.ptr; S.luts = c.d_luts.ptr; S.cand = c.d_cand.ptr; S.thr = c.d_thr.ptr; S.topk = c.d_topk.ptr;
    S.cnt = c.d_cnt.ptr; S.lo = nullptr; S.w_rows = w_rows; S.dim_pad = dim_pad; S.lut_pitch = lut_pitch; S.cap = cap; S.allow_tc = pages == 1;
    {
        ScanParams probe = base_scan_params(h, mode);
        plan.use_small = h->small_scan >= 0 && mode == TV_SCORE_PERMUTE_DOT && scan_small_supported(probe, int(nq), h->smem_limit);
    }

    // ---- inputs ----
    TV_CUDA(cudaStreamWaitEvent(st, h->ev_mut, 0));          // after every mutation enqueued on the handle's stream
    const float *dq = queries;
    if (!queries_on_device) {
        TV_CUDA(cudaMemcpyAsync(c.d_stage.ptr, queries, nq * dim * 4, cudaMemcpyHostToDevice, st));
        dq = c.d_stage.ptr;
    }
    DeviceFlags init{};
    init.first_invalid = ~0ull;
    init.first_unknown = ~0ull;
    *c.h_flags = init;
    TV_CUDA(cudaMemcpyAsync(c.d_flags, c.h_flags, sizeof(DeviceFlags), cudaMemcpyHostToDevice, st));
    TV_CUDA(cudaEventRecord(c.ev0, st));

    MaskOnDevice m;
    if (mask.prepared) {
        if (!h->prepared.valid) return fail(h, TV_ERR_INVALID_ARGUMENT, "no prepared mask: call tv_mask_prepare_* after the last change of the index");
        m.words = h->prepared.words.ptr; m.live = h->prepared.live.ptr;
        m.n_allowed = h->prepared.counts.ptr; m.n_live = reinterpret_cast<const uint32_t *>(h->prepared.counts.ptr + 1);
    } else if (mask.any()) {
        rc = build_mask(h, st, mask, c.d_mask, c.d_mask_bool, c.d_slots_in, c.d_live, c.d_allow_ids, &c.d_flags->first_unknown,
                        &c.d_flags->n_allowed, &c.d_flags->n_live, m);
        if (rc != TV_OK) return rc;
    }

    rc = enqueue_query_prep(h, st, S, plan, mode, dq, nq, &c.d_flags->first_invalid);
    if (rc != TV_OK) return rc;

    CandidateBuffers out_cb{};                                  // what finalize reads
    out_cb.topk = pages == 1 ? c.d_topk.ptr : c.d_keys_all.ptr;
    out_cb.k = int(kk);
    uint32_t *d_keff = &c.d_flags->k_eff;
    // decode / export of the finished rows, the status words and (host searches) the results, then one synchronisation
    auto finish = [&]() -> int {
        if (out_keys_dev) TV_CUDA(launch_export_keys(out_cb.topk, int64_t(nq * kk), key_offset, out_keys_dev, st));
        if (out_scores_dev) TV_CUDA(launch_finalize(out_cb, int(nq), m.n_allowed, int64_t(n), out_scores_dev, out_slots_dev, d_keff, 0, st));
        else TV_CUDA(launch_finalize(out_cb, int(nq), m.n_allowed, int64_t(n), c.d_scores.ptr, c.d_slots.ptr, d_keff, 1, st));
        h->launches++;
        TV_CUDA(cudaEventRecord(c.ev1, st));
        TV_CUDA(cudaMemcpyAsync(c.h_flags, c.d_flags, sizeof(DeviceFlags), cudaMemcpyDeviceToHost, st));
        if (!out_scores_dev && !out_keys_dev) {
            TV_CUDA(c.h_scores.reserve(nq * kk));
            TV_CUDA(c.h_slots.reserve(nq * kk));
            TV_CUDA(cudaMemcpyAsync(c.h_scores.ptr, c.d_scores.ptr, nq * kk * 4, cudaMemcpyDeviceToHost, st));
            TV_CUDA(cudaMemcpyAsync(c.h_slots.ptr, c.d_slots.ptr, nq * kk * 8, cudaMemcpyDeviceToHost, st));
        }
        TV_CUDA(cudaStreamSynchronize(st));
        float ms = 0.f;
        cudaEventElapsedTime(&ms, c.ev0, c.ev1);
        c.marks.collect();
        std::lock_guard<std::mutex> g(h->stat_mu);
        h->last_ms = ms; h->last_main_ms = c.marks.total_ms; h->last_main_launches = c.marks.launches;
        return TV_OK;
    };
    for (size_t page = 0; page < pages; ++page) {
        const size_t k_this = pages == 1 ? kk : std::min(kPageK, kk - page * kPageK);
        S.lo = page == 0 ? nullptr : c.d_floor.ptr;
        for (int attempt = 0; attempt < 2; ++attempt) {
            const bool careful = attempt == 1 || h->force_careful;
            rc = enqueue_search(h, st, &c.marks, S, plan, mode, nq, k_this, m, &c.d_flags->overflow, &c.d_flags->error, careful);
            if (rc != TV_OK) { c.marks.used = 0; return rc; }
            if (pages == 1) {
                rc = finish();                                  // the common case: one submission, one synchronisation
            } else {
                TV_CUDA(cudaMemcpyAsync(c.h_flags, c.d_flags, sizeof(DeviceFlags), cudaMemcpyDeviceToHost, st));
                TV_CUDA(cudaStreamSynchronize(st));
            }
            if (rc == TV_OK && mask.ids_host && c.h_flags->first_unknown != ~0ull) {     // id_map.rs:672-677
                const uint64_t bad = mask.ids_host[c.h_flags->first_unknown];
                { std::lock_guard<std::mutex> g(h->stat_mu); h->err_id = bad; }
                rc = fail(h, TV_ERR_UNKNOWN_ID, "allowlist id " + std::to_string(bad) + " is not in the index");
            }
            if (rc == TV_OK) rc = check_flags(h, c.h_flags, queries, queries_on_device, st);
            if (rc != TV_OK) { c.marks.used = 0; return rc; }
            if (!c.h_flags->overflow) break;
            if (careful) return fail(h, TV_ERR_CUDA, "candidate overflow in the bounded schedule (internal error)");
            // a chunk produced more candidates than the buffer holds: redo this page with bounded chunks
            c.h_flags->overflow = 0;
            TV_CUDA(cudaMemcpyAsync(&c.d_flags->overflow, &c.h_flags->overflow, 4, cudaMemcpyHostToDevice, st));
        }
        if (pages > 1) {
            // this page's keys into their columns of the full rows; its last key bounds the next page from below
            TV_CUDA(cudaMemcpy2DAsync(c.d_keys_all.ptr + page * kPageK, kk * 8, c.d_topk.ptr, k_this * 8, k_this * 8, nq,
                                      cudaMemcpyDeviceToDevice, st));
            if (page + 1 < pages) {
                TV_CUDA(launch_advance_floor(c.d_thr.ptr, c.d_floor.ptr, int(nq), st));
            } else {
                rc = finish();
                if (rc != TV_OK) return rc;
            }
        }
    }
    *k_eff_out = c.h_flags->k_eff;
    return TV_OK;
}

// Shared front end of the host-memory search entry points (validation order of lib.rs:1345-1433).
int search_host(tv_index *h, const float *queries, size_t nq, size_t dim, size_t k, const MaskSpec &mask,
                float *scores_out, int64_t *slots_out, uint64_t *ids_out, size_t *k_eff) {
    if (k_eff) *k_eff = 0;
    if (h->dim == 0) return TV_OK;                                   // lazy index: empty result
    if (dim != h->dim)
        return fail(h, TV_ERR_QUERY_BUFFER_NOT_MULTIPLE_OF_DIM, "query dimension " + std::to_string(dim) + " does not match index dim " + std::to_string(h->dim));
    if (h->n == 0) {
        if (mask.bool_host && mask.bool_len != 0)
            return fail(h, TV_ERR_MASK_LENGTH_MISMATCH, "mask length " + std::to_string(mask.bool_len) + " does not match index length 0");
        return TV_OK;
    }
    if (mask.bool_host && mask.bool_len != h->n)
        return fail(h, TV_ERR_MASK_LENGTH_MISMATCH, "mask length " + std::to_string(mask.bool_len) + " does not match index length " + std::to_string(h->n));
    if (mask.words_host && mask.n_words != (h->n + 63) / 64)
        return fail(h, TV_ERR_MASK_LENGTH_MISMATCH, "mask has " + std::to_string(mask.n_words) + " words, index needs " + std::to_string((h->n + 63) / 64));
    if (nq == 0) {
        // no queries: empty result whose row width is still min(k, len, n_allowed) (lib.rs:1460)
        size_t allowed = h->n;
        if (mask.bool_host) {
            allowed = 0;
            for (size_t i = 0; i < h->n; ++i) allowed += mask.bool_host[i] != 0;
        } else if (mask.words_host) {
            allowed = 0;
            for (size_t i = 0; i < h->n; ++i) allowed += (mask.words_host[i >> 6] >> (i & 63)) & 1ull;
        } else if (mask.slots_host) {
            std::unordered_set<uint32_t> distinct(mask.slots_host, mask.slots_host + mask.n_slots);
            allowed = distinct.size();
        }
        if (k_eff) *k_eff = std::min(std::min(k, h->n), allowed);
        return TV_OK;
    }
    size_t ke = 0;
    CtxLease lease(h);
    SearchCtx &c = *lease.c;
    int rc = search_core(h, c, queries, false, nq, k, mask, nullptr, nullptr, &ke);
    if (rc != TV_OK) return rc;
    const size_t kk = std::min(k, h->n);
    for (size_t q = 0; q < nq; ++q) {
        std::memcpy(scores_out + q * ke, c.h_scores.ptr + q * kk, ke * sizeof(float));
        if (slots_out) std::memcpy(slots_out + q * ke, c.h_slots.ptr + q * kk, ke * sizeof(int64_t));
        if (ids_out)
            for (size_t j = 0; j < ke; ++j) ids_out[q * ke + j] = h->slot_to_id[size_t(c.h_slots.ptr[q * kk + j])];   // id_map.rs:695-705
    }
    if (k_eff) *k_eff = ke;
    return TV_OK;
}

// Allowlist ids -> slots (id_map.rs:670-683): one hash lookup per id; large lists are split over host threads (lookups
// only read the table) and the first unknown id in list order is the one reported, as in a sequential walk.
int resolve_allowlist(tv_index *h, const uint64_t *allow_ids, size_t n_allow, std::vector<uint32_t> &slots) {
    if (n_allow == 0) return fail(h, TV_ERR_ALLOWLIST_EMPTY, "allowlist is empty");
    slots.resize(n_allow);
    const size_t n_threads = n_allow < (size_t(1) << 16) ? 1 : std::min<size_t>(16, std::max(1u, std::thread::hardware_concurrency()));
    std::vector<size_t> first_unknown(n_threads, n_allow);
    auto resolve = [&](size_t t) {
        const size_t lo = n_allow * t / n_threads, hi = n_allow * (t + 1) / n_threads;
        for (size_t i = lo; i < hi; ++i) {
            auto it = h->id_to_slot.find(allow_ids[i]);
            if (it == h->id_to_slot.end()) { first_unknown[t] = i; return; }
            slots[i] = it->second;
        }
    };
    if (n_threads == 1) {
        resolve(0);
    } else {
        std::vector<std::thread> pool;
        for (size_t t = 0; t < n_threads; ++t) pool.emplace_back(resolve, t);
        for (auto &th : pool) th.join();
    }
    const size_t bad = *std::min_element(first_unknown.begin(), first_unknown.end());
    if (bad < n_allow) {
        { std::lock_guard<std::mutex> g(h->stat_mu); h->err_id = allow_ids[bad]; }
        return fail(h, TV_ERR_UNKNOWN_ID, "allowlist id " + std::to_string(allow_ids[bad]) + " is not in the index");
    }
    return TV_OK;
}

// ---- host layout conversion for import / export (pack.rs:264-334, 375-467) ----
void packed_to_blocked(const uint8_t *packed, size_t n, int bits, int dim, std::vector<uint8_t> &blocked) {
    const int bpp = dim / 8, cpb = 8 / bits, ng = dim / cpb, bpr = bits * bpp, field = bits == 3 ? 4 : bits;
    blocked.assign(((n + 31) / 32) * size_t(ng) * 32, 0);
    for (size_t v = 0; v < n; ++v) {
        const uint8_t *row = packed + v * bpr;
        uint8_t *out = blocked.data() + (v / 32) * size_t(ng) * 32 + (v % 32);
        for (int j = 0; j < dim; ++j) {
            int code = 0;
            for (int p = 0; p < bits; ++p) code |= ((row[p * bpp + j / 8] >> (7 - j % 8)) & 1) << p;
            out[size_t(j / cpb) * 32] |= uint8_t(code << ((cpb - 1 - j % cpb) * field));
        }
    }
}
void blocked_to_packed(const uint8_t *blocked, size_t n, int bits, int dim, uint8_t *packed) {
    const int bpp = dim / 8, cpb = 8 / bits, ng = dim / cpb, bpr = bits * bpp, field = bits == 3 ? 4 : bits;
    std::memset(packed, 0, n * size_t(bpr));
    for (size_t v = 0; v < n; ++v) {
        uint8_t *row = packed + v * bpr;
        const uint8_t *in = blocked + (v / 32) * size_t(ng) * 32 + (v % 32);
        for (int j = 0; j < dim; ++j) {
            const int code = (in[size_t(j / cpb) * 32] >> ((cpb - 1 - j % cpb) * field)) & ((1 << bits) - 1);
            for (int p = 0; p < bits; ++p) row[p * bpp + j / 8] |= uint8_t(((code >> p) & 1) << (7 - j % 8));
        }
    }
}

}  // namespace

// =====================================================================================================
// C ABI
// =====================================================================================================
extern "C" {

const char *tv_version(void) { return "turbovec_b200 0.1 (sm_100a)"; }

int tv_exchange_layout_conflicts(size_t dim, int *store_plain, int *gather_plain, int *store_layout, int *gather_layout) {
    if (!store_plain || !gather_plain || !store_layout || !gather_layout) return TV_ERR_INVALID_ARGUMENT;
    if (dim == 0 || dim % 32 != 0 || dim > size_t(kMaxDim)) return TV_ERR_UNSUPPORTED;
    const RotationTables rot = build_rotation_tables(int(dim));
    ExchangeLayoutHost ex;
    if (!build_exchange_layout(int(dim), rot.packed[1].data(), ex)) return TV_ERR_UNSUPPORTED;
    exchange_layout_conflicts(int(dim), rot.packed[1].data(), nullptr, store_plain, gather_plain);
    exchange_layout_conflicts(int(dim), rot.packed[1].data(), &ex, store_layout, gather_layout);
    return TV_OK;
}

int tv_quantise_grid_lookup(const float *boundaries, int count, const float *values, size_t n, uint8_t *codes_out) {
    if (!boundaries || (n && (!values || !codes_out))) return TV_ERR_INVALID_ARGUMENT;
    QuantGridHost grid;
    if (!build_quant_grid(boundaries, count, grid)) return TV_ERR_UNSUPPORTED;
    for (size_t i = 0; i < n; ++i) codes_out[i] = uint8_t(quant_grid_code(grid, values[i]));
    return TV_OK;
}

int tv_index_create(size_t dim, int bit_width, int kind, int device, tv_index **out) {
    tv_index *h = nullptr;
    if (!out) return fail(h, TV_ERR_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    if (bit_width < 2 || bit_width > 4) return fail(h, TV_ERR_BIT_WIDTH_OUT_OF_RANGE, "bit_width must be 2, 3 or 4, got " + std::to_string(bit_width));
    if (dim != 0) {
        if (dim % 8 != 0) return fail(h, TV_ERR_DIM_NOT_POSITIVE_MULTIPLE_OF_8, "dim must be a positive multiple of 8, got " + std::to_string(dim));
        if (dim > size_t(kMaxDim)) return fail(h, TV_ERR_DIM_TOO_LARGE, "dim " + std::to_string(dim) + " exceeds " + std::to_string(kMaxDim));
    }
    if (kind != TV_KIND_POSITIONAL && kind != TV_KIND_IDMAP) return fail(h, TV_ERR_INVALID_ARGUMENT, "unknown index kind");
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(h, TV_ERR_CUDA, std::string("no CUDA device: this library has no CPU path (") + cudaGetErrorString(e) + ")");
    }
    if (device < 0 || device >= count) return fail(h, TV_ERR_INVALID_ARGUMENT, "device ordinal out of range");
    h = new tv_index();
    h->kind = kind; h->bits = bit_width; h->device = device; h->dim = dim;
    auto bail = [&](const char *what, cudaError_t err) {
        std::string msg = std::string(what) + ": " + cudaGetErrorString(err);
        cudaGetLastError();
        delete h;
        g_create_error = msg;
        return int(TV_ERR_CUDA);
    };
    if ((e = cudaSetDevice(device)) != cudaSuccess) return bail("cudaSetDevice", e);
    cudaDeviceProp prop{};
    if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) return bail("cudaGetDeviceProperties", e);
    h->sm_count = prop.multiProcessorCount;
    h->smem_limit = prop.sharedMemPerBlockOptin;
    if ((e = cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking)) != cudaSuccess) return bail("cudaStreamCreate", e);
    if ((e = cudaEventCreate(&h->ev0)) != cudaSuccess) return bail("cudaEventCreate", e);
    if ((e = cudaEventCreate(&h->ev1)) != cudaSuccess) return bail("cudaEventCreate", e);
    if ((e = cudaEventCreateWithFlags(&h->ev_mut, cudaEventDisableTiming)) != cudaSuccess) return bail("cudaEventCreate", e);
    if ((e = cudaEventRecord(h->ev_mut, h->stream)) != cudaSuccess) return bail("cudaEventRecord", e);
    if ((e = cudaMalloc(&h->d_flags, sizeof(DeviceFlags))) != cudaSuccess) return bail("cudaMalloc", e);
    if ((e = cudaMallocHost(&h->h_flags, sizeof(DeviceFlags))) != cudaSuccess) return bail("cudaMallocHost", e);
    for (int i = 0; i < kSearchCtxs; ++i)
        if ((e = h->ctx[i].init()) != cudaSuccess) return bail("search context", e);
    *out = h;
    return TV_OK;
}

void tv_index_destroy(tv_index *h) { delete h; }

const char *tv_last_error(const tv_index *h) { return h ? h->last_error.c_str() : g_create_error.c_str(); }

void tv_error_detail(const tv_index *h, size_t *vector_index, size_t *coord_index, float *value, uint64_t *id) {
    if (!h) return;
    if (vector_index) *vector_index = h->err_vec;
    if (coord_index) *coord_index = h->err_coord;
    if (value) *value = h->err_value;
    if (id) *id = h->err_id;
}

size_t tv_len(const tv_index *h) {
    if (!h) return 0;
    std::shared_lock<std::shared_mutex> lock(const_cast<tv_index *>(h)->mu);
    return h->n;
}
size_t tv_dim(const tv_index *h) { return h ? h->dim : 0; }
int tv_bit_width(const tv_index *h) { return h ? h->bits : 0; }
int tv_kind(const tv_index *h) { return h ? h->kind : -1; }
uint64_t tv_launch_count(const tv_index *h) { return h ? h->launches.load() : uint64_t(0); }
float tv_last_kernel_ms(const tv_index *h) { return h ? h->last_ms : 0.f; }
float tv_last_main_kernel_ms(const tv_index *h, int *launches) {
    if (!h) return 0.f;
    if (launches) *launches = h->last_main_launches;
    return h->last_main_ms;
}

int tv_set_option(tv_index *h, int option, int64_t value) {
    if (!h) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    switch (option) {
        case TV_OPT_SCORE_MODE:
            if (value < TV_SCORE_AUTO || value > TV_SCORE_LUT_FLUSH) return fail(h, TV_ERR_INVALID_ARGUMENT, "unknown score mode");
            if (value == TV_SCORE_PERMUTE_DOT && h->bits != 4) return fail(h, TV_ERR_INVALID_ARGUMENT, "permute-dot scoring needs 4-bit codes");
            h->score_mode = int(value);
            return TV_OK;
        case TV_OPT_MMA_MIN_BATCH: h->mma_min_batch = value; return TV_OK;
        case TV_OPT_FORCE_CAREFUL: h->force_careful = value != 0; return TV_OK;
        case TV_OPT_TC_TILES: h->tc_tiles = value == 1 ? 1 : 2; return TV_OK;
        case TV_OPT_INGEST_PIPELINE: h->ingest_pipeline = value < 0 || value > 2 ? 1 : int(value); return TV_OK;
        case TV_OPT_PD_SPLIT: h->pd_split = value != 0; return TV_OK;
        case TV_OPT_SMALL_SCAN: h->small_scan = value < 0 ? -1 : int(value & 7); return TV_OK;
        case TV_OPT_FAIL_NEXT: h->fail_next = value < 0 ? 0 : int(value); return TV_OK;
        case TV_OPT_TC_WIDE: h->tc_wide = value != 0; return TV_OK;
        case TV_OPT_DENSE_PAIR: h->dense_pair = value != 0; return TV_OK;
        case TV_OPT_TC_EXPANDED:
            h->tc_expanded = value < 0 || value > 2 ? 1 : int(value);
            if (h->tc_expanded == 0) { std::lock_guard<std::mutex> g(h->expanded.mu); h->expanded.drop(); }
            return TV_OK;
        default: return fail(h, TV_ERR_INVALID_ARGUMENT, "unknown option");
    }
}

int64_t tv_get_option(const tv_index *h, int option) {
    if (!h) return -1;
    switch (option) {
        case TV_OPT_SCORE_MODE: return h->dim ? resolve_mode(h) : h->score_mode;
        case TV_OPT_MMA_MIN_BATCH: return h->mma_min_batch;
        case TV_OPT_FORCE_CAREFUL: return h->force_careful;
        case TV_OPT_TC_TILES: return h->tc_tiles;
        case TV_OPT_INGEST_PIPELINE: return h->ingest_pipeline;
        case TV_OPT_PD_SPLIT: return h->pd_split;
        case TV_OPT_SMALL_SCAN: return h->small_scan;
        case TV_OPT_FAIL_NEXT: return h->fail_next;
        case TV_OPT_TC_WIDE: return h->tc_wide;
        case TV_OPT_TC_EXPANDED: return h->tc_expanded;
        case TV_OPT_DENSE_PAIR: return h->dense_pair;
        case TV_OPT_EXPANDED_BYTES: return h->expanded.levels.ptr ? int64_t(h->expanded.rows_cap * size_t(h->expanded.pitch)) : 0;
        default: return -1;
    }
}

int tv_add(tv_index *h, const float *vectors, size_t n, size_t dim) {
    if (!h || (!vectors && n)) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    if (h->kind != TV_KIND_POSITIONAL) return fail(h, TV_ERR_WRONG_INDEX_KIND, "tv_add on an id-mapped index; use tv_add_with_ids");
    return add_rows(h, vectors, n, dim, false);
}

int tv_add_device(tv_index *h, const float *vectors_device, size_t n, size_t dim) {
    if (!h || (!vectors_device && n)) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    if (h->kind != TV_KIND_POSITIONAL) return fail(h, TV_ERR_WRONG_INDEX_KIND, "tv_add_device on an id-mapped index");
    return add_rows(h, vectors_device, n, dim, true);
}

namespace {
int add_rows_with_ids(tv_index *h, const float *vectors, size_t n, size_t dim, const uint64_t *ids, bool on_device);
}
int tv_add_with_ids(tv_index *h, const float *vectors, size_t n, size_t dim, const uint64_t *ids) {
    return add_rows_with_ids(h, vectors, n, dim, ids, false);
}
int tv_add_with_ids_device(tv_index *h, const float *vectors_device, size_t n, size_t dim, const uint64_t *ids) {
    return add_rows_with_ids(h, vectors_device, n, dim, ids, true);
}
namespace {
int add_rows_with_ids(tv_index *h, const float *vectors, size_t n, size_t dim, const uint64_t *ids, bool on_device) {
    if (!h || (!vectors && n) || (!ids && n)) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    if (h->kind != TV_KIND_IDMAP) return fail(h, TV_ERR_WRONG_INDEX_KIND, "tv_add_with_ids needs an id-mapped index");
    if (dim == 0) return fail(h, TV_ERR_ZERO_DIM, "dim must be non-zero");          // id_map.rs:379-381
    // per id, in order: already present, then duplicate within the batch (id_map.rs:396-434)
    std::unordered_set<uint64_t> seen;
    seen.reserve(n * 2);
    for (size_t i = 0; i < n; ++i) {
        if (h->id_to_slot.count(ids[i])) {
            h->err_id = ids[i];
            return fail(h, TV_ERR_ID_ALREADY_PRESENT, "id " + std::to_string(ids[i]) + " is already present");
        }
        if (!seen.insert(ids[i]).second) {
            h->err_id = ids[i];
            return fail(h, TV_ERR_DUPLICATE_ID_IN_BATCH, "id " + std::to_string(ids[i]) + " appears twice in the batch");
        }
    }
    const size_t base = h->n;
    int rc = add_rows(h, vectors, n, dim, on_device);
    if (rc != TV_OK) return rc;
    h->slot_to_id.insert(h->slot_to_id.end(), ids, ids + n);
    h->id_to_slot.reserve(h->id_to_slot.size() + n);
    for (size_t i = 0; i < n; ++i) h->id_to_slot.emplace(ids[i], uint32_t(base + i));
    for (size_t i = 0; i < n; ++i) h->idtab.note(ids[i], uint32_t(base + i), h->slot_to_id.size());
    return TV_OK;
}
}  // namespace

int tv_swap_remove(tv_index *h, size_t slot, size_t *moved_from) {
    if (!h) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    if (h->kind != TV_KIND_POSITIONAL) return fail(h, TV_ERR_WRONG_INDEX_KIND, "tv_swap_remove on an id-mapped index; use tv_remove");
    if (slot >= h->n) return fail(h, TV_ERR_SLOT_OUT_OF_RANGE, "index " + std::to_string(slot) + " out of bounds (n_vectors = " + std::to_string(h->n) + ")");
    TV_CUDA(cudaSetDevice(h->device));
    const size_t last = h->n - 1;
    move_lane_kernel<<<(h->ngroups + 255) / 256, 256, 0, h->stream>>>(h->d_codes, h->d_scales, h->ngroups, int64_t(last), int64_t(slot));
    h->launches++;
    TV_CUDA(cudaGetLastError());
    // no synchronisation: the result is known on the host, and every later call on this handle runs on the
    // same stream, after the move
    h->mark_dirty(slot);                      // lib.rs:2879-2885: the hole and the moved-from slot diverge
    if (last != slot) h->mark_dirty(last);
    h->expanded.touch(slot);
    h->expanded.shrink(last);
    h->n = last;
    mutation_done(h);
    if (moved_from) *moved_from = last;
    return TV_OK;
}

int tv_remove(tv_index *h, uint64_t id, int *removed) {
    if (!h) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    if (removed) *removed = 0;
    if (h->kind != TV_KIND_IDMAP) return fail(h, TV_ERR_WRONG_INDEX_KIND, "tv_remove needs an id-mapped index");
    auto it = h->id_to_slot.find(id);
    if (it == h->id_to_slot.end()) return TV_OK;                       // id_map.rs:521-523
    const size_t slot = it->second, last = h->n - 1;
    TV_CUDA(cudaSetDevice(h->device));
    move_lane_kernel<<<(h->ngroups + 255) / 256, 256, 0, h->stream>>>(h->d_codes, h->d_scales, h->ngroups, int64_t(last), int64_t(slot));
    h->launches++;
    TV_CUDA(cudaGetLastError());
    h->mark_dirty(slot);
    if (last != slot) h->mark_dirty(last);
    h->expanded.touch(slot);
    h->expanded.shrink(last);
    h->n = last;                                                       // enqueued, not awaited (see tv_swap_remove)
    mutation_done(h);
    h->id_to_slot.erase(it);
    h->idtab.note(id, 0xffffffffu, h->slot_to_id.size());
    if (slot != last) {                                                // id_map.rs:557-561
        const uint64_t moved = h->slot_to_id[last];
        h->slot_to_id[slot] = moved;
        h->id_to_slot[moved] = uint32_t(slot);
        h->idtab.note(moved, uint32_t(slot), h->slot_to_id.size());
    }
    h->slot_to_id.pop_back();
    if (removed) *removed = 1;
    return TV_OK;
}

int tv_get_row(const tv_index *hc, size_t slot, uint8_t *groups_out, size_t capacity, float *scale_out) {
    tv_index *h = const_cast<tv_index *>(hc);
    if (!h || !groups_out || !scale_out) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    if (slot >= h->n) return fail(h, TV_ERR_SLOT_OUT_OF_RANGE, "index " + std::to_string(slot) + " out of bounds (n_vectors = " + std::to_string(h->n) + ")");
    if (capacity < size_t(h->ngroups)) return fail(h, TV_ERR_INVALID_ARGUMENT, "output buffer too small");
    TV_CUDA(cudaSetDevice(h->device));
    TV_CUDA(h->d_row.reserve(size_t(h->ngroups)));
    gather_row_kernel<<<(h->ngroups + 255) / 256, 256, 0, h->stream>>>(h->d_codes, h->ngroups, int64_t(slot), h->d_row.ptr);
    h->launches++;
    TV_CUDA(cudaGetLastError());
    TV_CUDA(cudaMemcpyAsync(groups_out, h->d_row.ptr, size_t(h->ngroups), cudaMemcpyDeviceToHost, h->stream));
    TV_CUDA(cudaMemcpyAsync(scale_out, h->d_scales + slot, 4, cudaMemcpyDeviceToHost, h->stream));
    TV_CUDA(cudaStreamSynchronize(h->stream));
    return TV_OK;
}

int tv_set_row(tv_index *h, size_t slot, const uint8_t *groups, size_t count, float scale) {
    if (!h || !groups) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    if (slot >= h->n) return fail(h, TV_ERR_SLOT_OUT_OF_RANGE, "index " + std::to_string(slot) + " out of bounds (n_vectors = " + std::to_string(h->n) + ")");
    if (count != size_t(h->ngroups)) return fail(h, TV_ERR_INVALID_ARGUMENT, "a row has " + std::to_string(h->ngroups) + " byte-groups, got " + std::to_string(count));
    if (!(scale >= 0.0f) || !std::isfinite(scale)) return fail(h, TV_ERR_PARTS_INVALID, "scale is negative or not finite");
    TV_CUDA(cudaSetDevice(h->device));
    TV_CUDA(h->d_row.reserve(count));
    TV_CUDA(cudaMemcpyAsync(h->d_row.ptr, groups, count, cudaMemcpyHostToDevice, h->stream));
    scatter_row_kernel<<<(h->ngroups + 255) / 256, 256, 0, h->stream>>>(h->d_codes, h->ngroups, int64_t(slot), h->d_row.ptr);
    h->launches++;
    TV_CUDA(cudaGetLastError());
    TV_CUDA(cudaMemcpyAsync(h->d_scales + slot, &scale, 4, cudaMemcpyHostToDevice, h->stream));
    TV_CUDA(cudaStreamSynchronize(h->stream));
    h->mark_dirty(slot);
    h->expanded.touch(slot);
    mutation_done(h);
    return TV_OK;
}

int tv_contains(const tv_index *h, uint64_t id, int *present) {
    if (!h || !present) return TV_ERR_INVALID_ARGUMENT;
    std::shared_lock<std::shared_mutex> lock(const_cast<tv_index *>(h)->mu);      // the tables move under a concurrent add / remove
    *present = h->id_to_slot.count(id) ? 1 : 0;
    return TV_OK;
}

int tv_ids(const tv_index *h, uint64_t *ids_out, size_t capacity) {
    if (!h || (!ids_out && capacity)) return TV_ERR_INVALID_ARGUMENT;
    std::shared_lock<std::shared_mutex> lock(const_cast<tv_index *>(h)->mu);
    if (capacity < h->slot_to_id.size()) return TV_ERR_INVALID_ARGUMENT;
    std::copy(h->slot_to_id.begin(), h->slot_to_id.end(), ids_out);
    return TV_OK;
}

int tv_search(tv_index *h, const float *queries, size_t nq, size_t dim, size_t k, const uint8_t *mask_bool,
              size_t mask_len, float *scores_out, int64_t *slots_out, size_t *k_eff) {
    if (!h || (!queries && nq)) return TV_ERR_INVALID_ARGUMENT;
    std::shared_lock<std::shared_mutex> lock(h->mu);
    MaskSpec m;
    m.bool_host = mask_bool; m.bool_len = mask_len;
    return search_host(h, queries, nq, dim, k, m, scores_out, slots_out, nullptr, k_eff);
}

int tv_search_mask_words(tv_index *h, const float *queries, size_t nq, size_t dim, size_t k, const uint64_t *mask_words,
                         size_t n_words, float *scores_out, int64_t *slots_out, size_t *k_eff) {
    if (!h || (!queries && nq)) return TV_ERR_INVALID_ARGUMENT;
    std::shared_lock<std::shared_mutex> lock(h->mu);
    MaskSpec m;
    m.words_host = mask_words; m.n_words = n_words;
    return search_host(h, queries, nq, dim, k, m, scores_out, slots_out, nullptr, k_eff);
}

int tv_search_allowlist(tv_index *h, const float *queries, size_t nq, size_t dim, size_t k, const uint64_t *allow_ids,
                        size_t n_allow, float *scores_out, uint64_t *ids_out, size_t *k_eff) {
    if (!h || (!queries && nq)) return TV_ERR_INVALID_ARGUMENT;
    std::shared_lock<std::shared_mutex> lock(h->mu);
    if (h->kind != TV_KIND_IDMAP) return fail(h, TV_ERR_WRONG_INDEX_KIND, "tv_search_allowlist needs an id-mapped index");
    if (k_eff) *k_eff = 0;
    MaskSpec m;
    std::vector<uint32_t> slots;
    if (allow_ids) {                                                    // id_map.rs:670-683
        if (n_allow == 0) return fail(h, TV_ERR_ALLOWLIST_EMPTY, "allowlist is empty");
        if (n_allow >= kDeviceAllowlistMin && !h->idtab.unusable && h->n > 0 && nq > 0) {
            m.ids_host = allow_ids; m.n_ids = n_allow;               // long lists: resolved by the device table
        } else {
            int rc = resolve_allowlist(h, allow_ids, n_allow, slots);
            if (rc != TV_OK) return rc;
            m.slots_host = slots.data(); m.n_slots = slots.size();
        }
    }
    return search_host(h, queries, nq, dim, k, m, scores_out, nullptr, ids_out, k_eff);
}

int tv_search_device(tv_index *h, const float *queries_device, size_t nq, size_t k, const uint64_t *mask_words_device,
                     float *scores_out_device, int64_t *slots_out_device, size_t *k_eff) {
    if (!h || (!queries_device && nq) || !scores_out_device || !slots_out_device) return TV_ERR_INVALID_ARGUMENT;
    std::shared_lock<std::shared_mutex> lock(h->mu);
    if (k_eff) *k_eff = 0;
    if (h->dim == 0 || h->n == 0 || nq == 0) return TV_OK;
    MaskSpec m;
    m.words_device = mask_words_device;
    size_t ke = 0;
    CtxLease lease(h);
    int rc = search_core(h, *lease.c, queries_device, true, nq, k, m, scores_out_device, slots_out_device, &ke);
    if (rc == TV_OK && k_eff) *k_eff = ke;
    return rc;
}

int tv_search_device_keys(tv_index *h, const float *queries_device, size_t nq, size_t k, const uint64_t *mask_words_device,
                          uint64_t slot_offset, uint64_t *keys_out_device, size_t *k_eff) {
    if (!h || (!queries_device && nq) || !keys_out_device) return TV_ERR_INVALID_ARGUMENT;
    std::shared_lock<std::shared_mutex> lock(h->mu);
    if (k_eff) *k_eff = 0;
    if (nq == 0 || k == 0) return TV_OK;
    if (slot_offset + h->n > 0x100000000ull) return fail(h, TV_ERR_UNSUPPORTED, "slot_offset + len exceeds 2^32: the key holds 32 slot bits");
    TV_CUDA(cudaSetDevice(h->device));
    CtxLease lease(h);
    SearchCtx &c = *lease.c;
    const size_t kk = std::min(k, h->n);
    if (h->dim == 0 || h->n == 0 || kk < k) {
        // rows are k wide whatever the shard holds: fill with empty keys first
        TV_CUDA(cudaMemsetAsync(keys_out_device, 0xff, nq * k * 8, c.stream));
        TV_CUDA(cudaStreamSynchronize(c.stream));
        if (h->dim == 0 || h->n == 0) return TV_OK;
    }
    MaskSpec m;
    m.words_device = mask_words_device;
    size_t ke = 0;
    int rc;
    if (kk == k) {
        rc = search_core(h, c, queries_device, true, nq, k, m, nullptr, nullptr, &ke, keys_out_device, slot_offset);
    } else {
        // fewer vectors than k: the search yields rows of kk keys; spread them over rows of k
        TV_CUDA(c.d_keys_tmp.reserve(nq * kk));
        rc = search_core(h, c, queries_device, true, nq, k, m, nullptr, nullptr, &ke, c.d_keys_tmp.ptr, slot_offset);
        if (rc == TV_OK) {
            TV_CUDA(cudaMemcpy2DAsync(keys_out_device, k * 8, c.d_keys_tmp.ptr, kk * 8, kk * 8, nq, cudaMemcpyDeviceToDevice, c.stream));
            TV_CUDA(cudaStreamSynchronize(c.stream));
        }
    }
    if (rc == TV_OK && k_eff) *k_eff = ke;
    return rc;
}

// ---- a mask kept on the device between searches -------------------------------------------------------
namespace {
int prepare_mask(tv_index *h, const MaskSpec &spec) {
    h->prepared.valid = false;
    if (h->dim == 0 || h->n == 0) return fail(h, TV_ERR_INVALID_ARGUMENT, "the index is empty: nothing to prepare a mask for");
    TV_CUDA(cudaSetDevice(h->device));
    TV_CUDA(h->prepared.counts.reserve(2));
    TV_CUDA(cudaMemsetAsync(h->prepared.counts.ptr, 0, 16, h->stream));
    MaskOnDevice m;
    TV_CUDA(cudaMemsetAsync(&h->d_flags->first_unknown, 0xff, 8, h->stream));
    int rc = build_mask(h, h->stream, spec, h->prepared.words, h->ctx[0].d_mask_bool, h->ctx[0].d_slots_in, h->prepared.live,
                        h->ctx[0].d_allow_ids, &h->d_flags->first_unknown,
                        h->prepared.counts.ptr, reinterpret_cast<uint32_t *>(h->prepared.counts.ptr + 1), m);
    if (rc != TV_OK) return rc;
    TV_CUDA(cudaEventRecord(h->ev_mut, h->stream));             // searches run on other streams: order them after this
    TV_CUDA(cudaMemcpyAsync(&h->h_flags->first_unknown, &h->d_flags->first_unknown, 8, cudaMemcpyDeviceToHost, h->stream));
    TV_CUDA(cudaStreamSynchronize(h->stream));
    if (spec.ids_host && h->h_flags->first_unknown != ~0ull) {
        const uint64_t bad = spec.ids_host[h->h_flags->first_unknown];
        { std::lock_guard<std::mutex> g(h->stat_mu); h->err_id = bad; }
        return fail(h, TV_ERR_UNKNOWN_ID, "allowlist id " + std::to_string(bad) + " is not in the index");
    }
    h->prepared.valid = true;
    return TV_OK;
}
}  // namespace

int tv_mask_prepare_device(tv_index *h, const uint64_t *mask_words_device) {
    if (!h || !mask_words_device) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    MaskSpec m;
    m.words_device = mask_words_device;
    return prepare_mask(h, m);
}

int tv_mask_prepare_words(tv_index *h, const uint64_t *mask_words, size_t n_words) {
    if (!h || !mask_words) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    if (n_words != (h->n + 63) / 64)
        return fail(h, TV_ERR_MASK_LENGTH_MISMATCH, "mask has " + std::to_string(n_words) + " words, index needs " + std::to_string((h->n + 63) / 64));
    MaskSpec m;
    m.words_host = mask_words; m.n_words = n_words;
    return prepare_mask(h, m);
}

int tv_mask_prepare_allowlist(tv_index *h, const uint64_t *allow_ids, size_t n_allow) {
    if (!h || !allow_ids) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    if (h->kind != TV_KIND_IDMAP) return fail(h, TV_ERR_WRONG_INDEX_KIND, "tv_mask_prepare_allowlist needs an id-mapped index");
    std::vector<uint32_t> slots;
    MaskSpec m;
    if (n_allow >= kDeviceAllowlistMin && !h->idtab.unusable && h->n > 0) {
        m.ids_host = allow_ids; m.n_ids = n_allow;
    } else {
        int rc = resolve_allowlist(h, allow_ids, n_allow, slots);
        if (rc != TV_OK) return rc;
        m.slots_host = slots.data(); m.n_slots = slots.size();
    }
    return prepare_mask(h, m);
}

int tv_search_prepared(tv_index *h, const float *queries, size_t nq, size_t dim, size_t k, float *scores_out,
                       int64_t *slots_out, uint64_t *ids_out, size_t *k_eff) {
    if (!h || (!queries && nq) || !scores_out) return TV_ERR_INVALID_ARGUMENT;
    std::shared_lock<std::shared_mutex> lock(h->mu);
    if (ids_out && h->kind != TV_KIND_IDMAP) return fail(h, TV_ERR_WRONG_INDEX_KIND, "ids are only available on an id-mapped index");
    if (k_eff) *k_eff = 0;
    if (!h->prepared.valid) return fail(h, TV_ERR_INVALID_ARGUMENT, "no prepared mask: call tv_mask_prepare_* after the last change of the index");
    if (nq == 0) return TV_OK;
    MaskSpec m;
    m.prepared = true;
    return search_host(h, queries, nq, dim, k, m, scores_out, slots_out, ids_out, k_eff);
}

int tv_search_device_prepared(tv_index *h, const float *queries_device, size_t nq, size_t k, float *scores_out_device,
                              int64_t *slots_out_device, size_t *k_eff) {
    if (!h || (!queries_device && nq) || !scores_out_device || !slots_out_device) return TV_ERR_INVALID_ARGUMENT;
    std::shared_lock<std::shared_mutex> lock(h->mu);
    if (k_eff) *k_eff = 0;
    if (!h->prepared.valid) return fail(h, TV_ERR_INVALID_ARGUMENT, "no prepared mask: call tv_mask_prepare_* after the last change of the index");
    if (nq == 0) return TV_OK;
    MaskSpec m;
    m.prepared = true;
    size_t ke = 0;
    CtxLease lease(h);
    int rc = search_core(h, *lease.c, queries_device, true, nq, k, m, scores_out_device, slots_out_device, &ke);
    if (rc == TV_OK && k_eff) *k_eff = ke;
    return rc;
}

int tv_merge_keys_device_chunked(int device, const uint64_t *keys_device, size_t n_lists, size_t nq, size_t k, size_t chunk_slots,
                                 float *scores_out_device, int64_t *slots_out_device, void *stream) {
    if (!keys_device || !scores_out_device || !slots_out_device) return TV_ERR_INVALID_ARGUMENT;
    if (n_lists == 0 || nq == 0 || k == 0) return TV_OK;
    if (n_lists * k > size_t(kMergeMaxKeys)) { g_create_error = "n_lists * k exceeds 8192 keys per query"; return TV_ERR_UNSUPPORTED; }
    if (chunk_slots > 0xffffffffull || chunk_slots % kBlock != 0) { g_create_error = "chunk_slots must be a multiple of 32 below 2^32"; return TV_ERR_INVALID_ARGUMENT; }
    if (cudaSetDevice(device) != cudaSuccess) { g_create_error = "cudaSetDevice failed"; return TV_ERR_CUDA; }
    cudaError_t e = launch_merge_keys(keys_device, int(n_lists), int(nq), int(k), uint32_t(chunk_slots), scores_out_device,
                                      slots_out_device, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) { g_create_error = std::string("merge kernel launch: ") + cudaGetErrorString(e); return TV_ERR_CUDA; }
    return TV_OK;
}

int tv_merge_keys_device(int device, const uint64_t *keys_device, size_t n_lists, size_t nq, size_t k, float *scores_out_device,
                         int64_t *slots_out_device, void *stream) {
    return tv_merge_keys_device_chunked(device, keys_device, n_lists, nq, k, 0, scores_out_device, slots_out_device, stream);
}

// -----------------------------------------------------------------------------------------------------
// Search without any allocation.
//
// Who needs it: code that runs where the CUDA allocator must not be touched — a serving loop with a hard
// latency limit (cudaMalloc takes a device-wide lock and may synchronise), a process whose memory pool
// has been handed out completely to other tenants, or a caller that has promised its framework "no
// allocator traffic after warm-up".  tv_search_device grows its scratch arrays on demand; this entry
// point instead keeps every byte of scratch in one fixed array that is part of the loaded library image.
//
// The array lives in device memory of every GPU that loads the library (kNoAllocScratchBytes each) until
// the process exits.  Its name is only a host-side handle: the device address is fetched once per device
// with cudaGetSymbolAddress and it is that address the kernels receive.
// -----------------------------------------------------------------------------------------------------
constexpr size_t kNoAllocMaxQueries = 8;
constexpr size_t kNoAllocMaxK = 128;
constexpr size_t kNoAllocMaxDim = 4096;
constexpr size_t kNoAllocCap = 4096;                     // candidate slots per query
constexpr size_t kNoAllocScratchBytes = 1280 * 1024;     // 1.25 MiB, layout below
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

namespace {
std::mutex g_noalloc_mu;                                 // one call at a time per process: the array is shared
void *g_noalloc_base[64] = {nullptr};                    // device address of the array, per device ordinal

struct NoAllocLayout {
    float *q_rot, *qscale, *qbias;
    int8_t *weights;
    uint32_t *wfrag;
    uint8_t *luts;
    uint64_t *cand, *thr, *topk;
    uint32_t *cnt;
};
NoAllocLayout carve_noalloc(unsigned char *base) {
    NoAllocLayout L;
    size_t off = 0;
    auto take = [&](size_t bytes) { unsigned char *p = base + off; off += (bytes + 255) & ~size_t(255); return p; };
    L.q_rot = reinterpret_cast<float *>(take(kNoAllocMaxQueries * kNoAllocMaxDim * 4));          // 128 KiB
    L.qscale = reinterpret_cast<float *>(take(16 * 4));
    L.qbias = reinterpret_cast<float *>(take(16 * 4));
    L.weights = reinterpret_cast<int8_t *>(take(16 * kNoAllocMaxDim));                           //  64 KiB
    L.wfrag = reinterpret_cast<uint32_t *>(take((kNoAllocMaxDim / 2 / 16) * 32 * 16));           //  64 KiB
    L.luts = reinterpret_cast<uint8_t *>(take(kNoAllocMaxQueries * (kNoAllocMaxDim / 2) * 32));  // 512 KiB
    L.cand = reinterpret_cast<uint64_t *>(take(kNoAllocMaxQueries * kNoAllocCap * 8));           // 256 KiB
    L.thr = reinterpret_cast<uint64_t *>(take(kNoAllocMaxQueries * 8));
    L.topk = reinterpret_cast<uint64_t *>(take(kNoAllocMaxQueries * kNoAllocMaxK * 8));          //   8 KiB
    L.cnt = reinterpret_cast<uint32_t *>(take(kNoAllocMaxQueries * 4));
    static_assert(kNoAllocMaxQueries * kNoAllocMaxDim * 4 + 16 * kNoAllocMaxDim + (kNoAllocMaxDim / 32) * 512 +
                          kNoAllocMaxQueries * (kNoAllocMaxDim / 2) * 32 + kNoAllocMaxQueries * kNoAllocCap * 8 +
                          kNoAllocMaxQueries * kNoAllocMaxK * 8 + 8 * 256 <= kNoAllocScratchBytes,
                  "scratch layout exceeds the static array");
    return L;
}
}  // namespace

int tv_search_device_noalloc(tv_index *h, const float *queries_device, size_t nq, size_t k, float *scores_out_device,
                             int64_t *slots_out_device, size_t *k_eff) {
    if (!h || (!queries_device && nq) || !scores_out_device || !slots_out_device) return TV_ERR_INVALID_ARGUMENT;
    std::shared_lock<std::shared_mutex> lock(h->mu);
    std::lock_guard<std::mutex> scratch_lock(g_noalloc_mu);
    if (k_eff) *k_eff = 0;
    if (nq > kNoAllocMaxQueries)
        return fail(h, TV_ERR_UNSUPPORTED, "tv_search_device_noalloc takes at most " + std::to_string(kNoAllocMaxQueries) + " queries per call, got " + std::to_string(nq));
    if (k > kNoAllocMaxK)
        return fail(h, TV_ERR_UNSUPPORTED, "tv_search_device_noalloc takes k up to " + std::to_string(kNoAllocMaxK) + ", got " + std::to_string(k));
    if (h->dim > kNoAllocMaxDim)
        return fail(h, TV_ERR_UNSUPPORTED, "tv_search_device_noalloc supports dim up to " + std::to_string(kNoAllocMaxDim) + ", index has " + std::to_string(h->dim));
    if (h->dim == 0 || h->n == 0 || nq == 0 || k == 0) return TV_OK;
    if (!h->tables_ready) return fail(h, TV_ERR_INVALID_ARGUMENT, "index tables are not built yet: call tv_prepare (or add rows) before tv_search_device_noalloc");
    if (h->device < 0 || h->device >= 64) return fail(h, TV_ERR_UNSUPPORTED, "device ordinal above 63");
    TV_CUDA(cudaSetDevice(h->device));
    if (g_noalloc_base[h->device] == nullptr) {
        // one-time set-up on this device (device current): resolve the array's device address
        void *ptr = nullptr;
        TV_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
        g_noalloc_base[h->device] = ptr;
    }
    const NoAllocLayout L = carve_noalloc(static_cast<unsigned char *>(g_noalloc_base[h->device]));

    const size_t n = h->n;
    const int ng = h->ngroups, mode = resolve_mode(h);
    const size_t kk = std::min(k, n);
    // The CUDA-core kernels only: their launches need nothing beyond the fixed array.  Geometries whose u8 tables
    // do not fit in shared memory even for one query have no such kernel.
    ScanPlan plan;
    int rc = plan_scan(h, mode, nq, false, plan);
    if (rc != TV_OK) return rc;

    SearchScratch S{};
    S.q_rot = L.q_rot; S.qscale = L.qscale; S.qbias = L.qbias; S.weights = L.weights; S.wfrag = L.wfrag; S.luts = L.luts;
    S.cand = L.cand; S.thr = L.thr; S.topk = L.topk; S.cnt = L.cnt; S.lo = nullptr;
    S.w_rows = 16; S.dim_pad = kNoAllocMaxDim; S.lut_pitch = size_t((ng + 3) / 4 * 4) * 32; S.cap = int(kNoAllocCap); S.allow_tc = false;
    {
        ScanParams probe = base_scan_params(h, mode);
        // (the tensor map of the swizzled variants is built on the host stack: no allocation)
        plan.use_small = h->small_scan >= 0 && mode == TV_SCORE_PERMUTE_DOT && scan_small_supported(probe, int(nq), h->smem_limit);
    }

    // the context supplies a stream and the status words (allocated when the handle was created)
    CtxLease lease(h);
    SearchCtx &c = *lease.c;
    cudaStream_t st = c.stream;
    TV_CUDA(cudaStreamWaitEvent(st, h->ev_mut, 0));
    DeviceFlags init{};
    init.first_invalid = ~0ull;
    *c.h_flags = init;
    TV_CUDA(cudaMemcpyAsync(c.d_flags, c.h_flags, sizeof(DeviceFlags), cudaMemcpyHostToDevice, st));
    TV_CUDA(cudaEventRecord(c.ev0, st));

    // The array still holds the previous call's data.  Query preparation clears the query operands it does not
    // overwrite, and the schedule resets counters, thresholds and result keys at its start.
    rc = enqueue_query_prep(h, st, S, plan, mode, queries_device, nq, &c.d_flags->first_invalid);
    if (rc != TV_OK) return rc;
    MaskOnDevice no_mask;
    CandidateBuffers out_cb{};
    out_cb.topk = L.topk; out_cb.k = int(kk);
    // The same geometric chunk schedule as tv_search_device (a few launches for any index size).  If a chunk
    // overflows a candidate list (adversarial order), the search is redone with chunks of at most the list's
    // capacity, which cannot overflow; neither schedule needs memory beyond the fixed array.
    for (int attempt = 0; attempt < 2; ++attempt) {
        const bool careful = attempt == 1 || h->force_careful;
        rc = enqueue_search(h, st, &c.marks, S, plan, mode, nq, kk, no_mask, &c.d_flags->overflow, &c.d_flags->error, careful);
        if (rc != TV_OK) { c.marks.used = 0; return rc; }
        TV_CUDA(launch_finalize(out_cb, int(nq), nullptr, int64_t(n), scores_out_device, slots_out_device, &c.d_flags->k_eff, 0, st));
        h->launches++;
        TV_CUDA(cudaEventRecord(c.ev1, st));
        TV_CUDA(cudaMemcpyAsync(c.h_flags, c.d_flags, sizeof(DeviceFlags), cudaMemcpyDeviceToHost, st));
        TV_CUDA(cudaStreamSynchronize(st));
        {
            float ms = 0.f;
            cudaEventElapsedTime(&ms, c.ev0, c.ev1);
            c.marks.collect();
            std::lock_guard<std::mutex> g(h->stat_mu);
            h->last_ms = ms; h->last_main_ms = c.marks.total_ms; h->last_main_launches = c.marks.launches;
        }
        rc = check_flags(h, c.h_flags, queries_device, true, st);
        if (rc != TV_OK) return rc;
        if (!c.h_flags->overflow) break;
        if (careful) return fail(h, TV_ERR_CUDA, "candidate overflow in the bounded schedule (internal error)");
        c.h_flags->overflow = 0;
        TV_CUDA(cudaMemcpyAsync(&c.d_flags->overflow, &c.h_flags->overflow, 4, cudaMemcpyHostToDevice, st));
    }
    if (k_eff) *k_eff = c.h_flags->k_eff;
    return TV_OK;
}

int tv_measure_int8_peak_for(int device, double seconds, double *ops_per_second) {
    if (!ops_per_second) return TV_ERR_INVALID_ARGUMENT;
    *ops_per_second = 0.0;
    cudaDeviceProp prop{};
    if (cudaSetDevice(device) != cudaSuccess || cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
        cudaGetLastError();
        g_create_error = "tv_measure_int8_peak: no such CUDA device";
        return TV_ERR_CUDA;
    }
    *ops_per_second = measure_int8_peak(prop.multiProcessorCount, seconds, nullptr);
    if (*ops_per_second <= 0.0) { g_create_error = "tv_measure_int8_peak: the measurement kernel failed"; return TV_ERR_CUDA; }
    return TV_OK;
}

int tv_measure_int8_peak(int device, double *ops_per_second) { return tv_measure_int8_peak_for(device, 0.0, ops_per_second); }

int tv_prepare(tv_index *h) {
    if (!h) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    if (h->dim == 0) return TV_OK;
    TV_CUDA(cudaSetDevice(h->device));
    return ensure_tables(h);
}

size_t tv_blocked_bytes(const tv_index *h) {
    if (!h || h->dim == 0) return 0;
    return ((h->n + kBlock - 1) / kBlock) * size_t(h->dim / (8 / h->bits)) * kBlock;
}

int tv_export_blocked(const tv_index *hc, uint8_t *blocked_out, size_t blocked_capacity, float *scales_out, size_t scales_capacity) {
    tv_index *h = const_cast<tv_index *>(hc);
    if (!h) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    const size_t bytes = tv_blocked_bytes(h);
    if ((blocked_out && blocked_capacity < bytes) || (scales_out && scales_capacity < h->n)) return fail(h, TV_ERR_INVALID_ARGUMENT, "output buffer too small");
    if (h->n == 0) return TV_OK;
    TV_CUDA(cudaSetDevice(h->device));
    if (blocked_out) TV_CUDA(cudaMemcpyAsync(blocked_out, h->d_codes, bytes, cudaMemcpyDeviceToHost, h->stream));
    if (scales_out) TV_CUDA(cudaMemcpyAsync(scales_out, h->d_scales, h->n * 4, cudaMemcpyDeviceToHost, h->stream));
    TV_CUDA(cudaStreamSynchronize(h->stream));
    return TV_OK;
}

int tv_export_packed(const tv_index *hc, uint8_t *packed_out, size_t capacity) {
    tv_index *h = const_cast<tv_index *>(hc);
    if (!h) return TV_ERR_INVALID_ARGUMENT;
    size_t n, dim, blocked_bytes;
    {
        // a consistent view of the sizes; the export below takes the lock itself and refuses a buffer that a
        // concurrent add has made too small
        std::shared_lock<std::shared_mutex> lock(h->mu);
        n = h->n; dim = h->dim;
        blocked_bytes = tv_blocked_bytes(h);
    }
    if (n == 0) return TV_OK;
    const size_t need = n * size_t(h->bits) * dim / 8;
    if (!packed_out || capacity < need) return fail(h, TV_ERR_INVALID_ARGUMENT, "output buffer too small");
    std::vector<uint8_t> blocked(blocked_bytes);
    int rc = tv_export_blocked(h, blocked.data(), blocked.size(), nullptr, 0);
    if (rc != TV_OK) return rc;
    blocked_to_packed(blocked.data(), n, h->bits, int(dim), packed_out);
    return TV_OK;
}

int tv_import_packed(tv_index *h, size_t dim, const uint8_t *packed, size_t n, const float *scales, const uint64_t *ids) {
    if (!h || (n && (!packed || !scales))) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    if (h->n != 0) return fail(h, TV_ERR_PARTS_INVALID, "import needs an empty index");
    int rc = validate_dim_for_add(h, dim);
    if (rc != TV_OK) return rc;
    if ((h->kind == TV_KIND_IDMAP) != (ids != nullptr) && n) return fail(h, TV_ERR_PARTS_INVALID, "ids must be given exactly for id-mapped indexes");
    for (size_t i = 0; i < n; ++i)   // lib.rs:2460-2492: scales finite and non-negative
        if (!(scales[i] >= 0.0f) || !std::isfinite(scales[i])) return fail(h, TV_ERR_PARTS_INVALID, "scale " + std::to_string(i) + " is negative or not finite");
    if (ids) {
        std::unordered_set<uint64_t> seen(ids, ids + n);
        if (seen.size() != n) return fail(h, TV_ERR_PARTS_INVALID, "duplicate ids");
    }
    h->sync_bound = false;                     // the content is replaced: the next sync rewrites its file whole
    h->sync_path.clear();
    if (n == 0) { if (h->dim == 0) h->dim = dim; return TV_OK; }
    TV_CUDA(cudaSetDevice(h->device));
    const bool was_lazy = h->dim == 0;
    h->dim = dim;
    rc = ensure_tables(h);
    if (rc == TV_OK) rc = ensure_capacity(h, n);
    if (rc != TV_OK) { if (was_lazy) { h->dim = 0; h->tables_ready = false; } return rc; }
    std::vector<uint8_t> blocked;
    packed_to_blocked(packed, n, h->bits, int(dim), blocked);
    TV_CUDA(cudaMemcpyAsync(h->d_codes, blocked.data(), blocked.size(), cudaMemcpyHostToDevice, h->stream));
    TV_CUDA(cudaMemcpyAsync(h->d_scales, scales, n * 4, cudaMemcpyHostToDevice, h->stream));
    TV_CUDA(cudaStreamSynchronize(h->stream));
    h->n = n;
    h->expanded.reset();
    mutation_done(h);
    if (ids) {
        h->slot_to_id.assign(ids, ids + n);
        h->id_to_slot.clear();
        for (size_t i = 0; i < n; ++i) h->id_to_slot.emplace(ids[i], uint32_t(i));
        h->idtab.reset(h->slot_to_id);
    }
    return TV_OK;
}

// ---- v7 container: to_bytes / from_bytes / write / load (lib.rs:2167, 2207, 2055, 2235; io_v7.rs) ----
namespace {
int gather_parts(tv_index *h, V7Parts &p) {
    p.kind = h->kind; p.bits = h->bits; p.dim = h->dim; p.n = h->n;
    if (h->dim) {
        const Codebook &cb = h->tables_ready ? h->cb : codebook(h->bits, int(h->dim));
        p.boundaries = cb.boundaries; p.centroids = cb.centroids;
    } else {                                   // lazy index: the reference writes a zero placeholder codebook
        p.boundaries.assign((size_t(1) << h->bits) - 1, 0.f);
        p.centroids.assign(size_t(1) << h->bits, 0.f);
    }
    p.shift = h->shift; p.scale = h->scale_tq;
    p.blocked.resize(h->dim ? ((h->n + kBlock - 1) / kBlock) * size_t(h->dim / (8 / h->bits)) * kBlock : 0);
    p.scales.resize(h->n);
    if (h->n) {
        TV_CUDA(cudaSetDevice(h->device));
        TV_CUDA(cudaMemcpyAsync(p.blocked.data(), h->d_codes, p.blocked.size(), cudaMemcpyDeviceToHost, h->stream));
        TV_CUDA(cudaMemcpyAsync(p.scales.data(), h->d_scales, h->n * 4, cudaMemcpyDeviceToHost, h->stream));
        TV_CUDA(cudaStreamSynchronize(h->stream));
    }
    if (h->kind == TV_KIND_IDMAP) p.ids = h->slot_to_id;
    return TV_OK;
}
}  // namespace

uint32_t tv_crc32c(const uint8_t *data, size_t len) { return crc32c_split(data, len); }

size_t tv_image_bytes(const tv_index *h) {
    if (!h) return 0;
    std::shared_lock<std::shared_mutex> lock(const_cast<tv_index *>(h)->mu);
    V7Parts p;
    p.kind = h->kind; p.bits = h->bits; p.dim = h->dim; p.n = h->n; p.shift = h->shift;
    return v7_image_len(p);
}

int tv_to_bytes(const tv_index *hc, uint8_t *out, size_t capacity) {
    tv_index *h = const_cast<tv_index *>(hc);
    if (!h || !out) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    V7Parts p;
    int rc = gather_parts(h, p);
    if (rc != TV_OK) return rc;
    std::vector<uint8_t> img;
    v7_write_image(p, img);
    if (capacity < img.size()) return fail(h, TV_ERR_INVALID_ARGUMENT, "output buffer too small");
    std::memcpy(out, img.data(), img.size());
    return TV_OK;
}

namespace {
// `bind_path` non-null: the image was read from that file, and an index loaded from a file that a sync has
// claimed stays bound to it, so that its next sync writes only the delta (lib.rs load_v7).
int index_from_image(const uint8_t *data, size_t len, int expect_kind, int device, tv_index **out, const char *bind_path) {
    tv_index *h = nullptr;
    if (!data || !out) return fail(h, TV_ERR_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    V7Parts p;
    std::string err;
    if (!v7_read_image(data, len, p, err)) return fail(h, TV_ERR_PARTS_INVALID, err);
    if (p.kind != expect_kind)
        return fail(h, TV_ERR_WRONG_INDEX_KIND, p.kind == 1 ? "this v7 image holds an IdMapIndex" : "this v7 image holds a TurboQuantIndex");
    if (p.kind == 1) {
        std::unordered_set<uint64_t> seen(p.ids.begin(), p.ids.end());
        if (seen.size() != p.n) return fail(h, TV_ERR_PARTS_INVALID, "duplicate ids in the image");
    }
    int rc = tv_index_create(p.dim, p.bits, p.kind, device, &h);
    if (rc != TV_OK) return rc;
    auto bail = [&](int code) { g_create_error = h->last_error; delete h; return code; };
    if (p.dim == 0) { *out = h; return TV_OK; }
    if (cudaSetDevice(h->device) != cudaSuccess) return bail(TV_ERR_CUDA);
    h->shift = p.shift; h->scale_tq = p.scale;
    rc = ensure_tables(h);
    if (rc != TV_OK) return bail(rc);
    if (p.boundaries != h->cb.boundaries || p.centroids != h->cb.centroids) {
        // the image carries the codebook it was encoded against; it wins over a re-solve (io_v7.rs load)
        h->cb.boundaries = p.boundaries; h->cb.centroids = p.centroids;
        rc = upload_codebook(h);
        if (rc != TV_OK) return bail(rc);
    }
    rc = upload_calibration(h);
    if (rc == TV_OK && p.n) rc = ensure_capacity(h, p.n);
    if (rc != TV_OK) return bail(rc);
    if (p.n) {
        if (cudaMemcpyAsync(h->d_codes, p.blocked.data(), p.blocked.size(), cudaMemcpyHostToDevice, h->stream) != cudaSuccess ||
            cudaMemcpyAsync(h->d_scales, p.scales.data(), p.n * 4, cudaMemcpyHostToDevice, h->stream) != cudaSuccess ||
            cudaStreamSynchronize(h->stream) != cudaSuccess) {
            h->last_error = "upload of the image failed";
            return bail(TV_ERR_CUDA);
        }
    }
    h->n = p.n;
    if (p.kind == 1) {
        h->slot_to_id = p.ids;
        for (size_t i = 0; i < p.n; ++i) h->id_to_slot.emplace(p.ids[i], uint32_t(i));
        h->idtab.reset(h->slot_to_id);
    }
    if (bind_path && p.nonce != 0) {           // an unclaimed snapshot is loaded unbound: the first sync claims it
        h->sync_bound = true;
        h->sync_path = bind_path;
        h->sync_cursor = V7Cursor{p.gen, uint64_t(p.n), h->calib_gen, p.nonce};
        h->sync_pending.insert(p.pending_slots.begin(), p.pending_slots.end());
    }
    *out = h;
    return TV_OK;
}
}  // namespace

int tv_from_bytes(const uint8_t *data, size_t len, int expect_kind, int device, tv_index **out) {
    return index_from_image(data, len, expect_kind, device, out, nullptr);
}

// Atomic replace: write a temp file beside the destination, fsync it, rename over it (io.rs:14-27).
int tv_write(const tv_index *hc, const char *path) {
    tv_index *h = const_cast<tv_index *>(hc);
    if (!h || !path) return TV_ERR_INVALID_ARGUMENT;
    std::vector<uint8_t> img(tv_image_bytes(h));
    int rc = tv_to_bytes(h, img.data(), img.size());
    if (rc != TV_OK) return rc;
    std::string err;
    if (!v7_write_file_atomic(path, img.data(), img.size(), err)) return fail(h, TV_ERR_IO, err);
    return TV_OK;
}

int tv_load(const char *path, int expect_kind, int device, tv_index **out) {
    tv_index *h = nullptr;
    if (!path || !out) return fail(h, TV_ERR_INVALID_ARGUMENT, "null argument");
    FILE *f = std::fopen(path, "rb");
    if (!f) return fail(h, TV_ERR_IO, std::string("cannot open ") + path);
    std::fseek(f, 0, SEEK_END);
    const long sz = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    std::vector<uint8_t> buf(sz > 0 ? size_t(sz) : 0);
    const bool ok = std::fread(buf.data(), 1, buf.size(), f) == buf.size();
    std::fclose(f);
    if (!ok) return fail(h, TV_ERR_IO, std::string("cannot read ") + path);
    return index_from_image(buf.data(), buf.size(), expect_kind, device, out, path);
}

// Incremental persistence (lib.rs sync :1737, sync_v7_impl :1813-1955).
int tv_sync(tv_index *h, const char *path) {
    if (!h || !path) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    if (h->dim == 0) return fail(h, TV_ERR_DIM_NOT_SET, "cannot sync a lazy index that has never seen an add or calibrate");
    int rc = ensure_tables(h);
    if (rc != TV_OK) return rc;
    TV_CUDA(cudaSetDevice(h->device));
    const size_t rb = size_t(h->ngroups);
    V7SyncSource src;
    src.kind = h->kind; src.bits = h->bits; src.dim = h->dim; src.n = h->n; src.n_calib = h->shift.size();
    src.ids = h->kind == TV_KIND_IDMAP ? h->slot_to_id.data() : nullptr;

    // The identity check runs whenever this index is bound to the path, also when a calibration has queued
    // a compaction: a rewrite over a file that another writer has taken over would destroy its commits.
    const bool bound = h->sync_bound && h->sync_path == path;
    V7CursorState state = V7_CURSOR_REPLACED;
    size_t stale_used = 0;
    std::string err;
    if (bound) {
        state = v7_cursor_state(path, h->sync_cursor, src, stale_used, err);
        if (state == V7_CURSOR_IO_ERROR) return fail(h, TV_ERR_IO, err);
        if (state == V7_CURSOR_FOREIGN)
            return fail(h, TV_ERR_SYNC_FOREIGN_FILE, std::string("the v7 file at ") + path + " no longer matches this index's last sync "
                        "(another writer advanced or replaced it); load the file to adopt its state, or choose a different path");
    }
    const bool incremental = bound && state == V7_CURSOR_INTACT && h->sync_cursor.calib_gen == h->calib_gen;
    auto unbind = [&]() {                      // a failed sync may have landed bytes: the next one rewrites whole
        h->sync_bound = false;
        h->sync_path.clear();
    };

    V7SyncPlan plan;
    if (incremental && v7_plan_sync(src, h->sync_cursor, h->sync_pending, h->sync_fresh, plan)) {
        // fetch the blocks the plan reads: runs of consecutive blocks, one copy each
        const std::vector<size_t> &need = plan.blocks_needed;
        std::vector<uint8_t> codes(need.size() * rb * kBlock);
        std::vector<float> scales(need.size() * kBlock, 0.0f);
        for (size_t i = 0; i < need.size();) {
            size_t j = i + 1;
            while (j < need.size() && need[j] == need[j - 1] + 1) ++j;
            const size_t first = need[i], rows_end = std::min(h->n, (need[j - 1] + 1) * kBlock);
            TV_CUDA(cudaMemcpyAsync(codes.data() + i * rb * kBlock, h->d_codes + first * rb * kBlock, (j - i) * rb * kBlock,
                                    cudaMemcpyDeviceToHost, h->stream));
            if (rows_end > first * kBlock)
                TV_CUDA(cudaMemcpyAsync(scales.data() + i * kBlock, h->d_scales + first * kBlock, (rows_end - first * kBlock) * 4,
                                        cudaMemcpyDeviceToHost, h->stream));
            i = j;
        }
        TV_CUDA(cudaStreamSynchronize(h->stream));
        src.block = [&](size_t block, const uint8_t *&c, const float *&sc) {
            const size_t i = size_t(std::lower_bound(need.begin(), need.end(), block) - need.begin());
            c = codes.data() + i * rb * kBlock;
            sc = scales.data() + i * kBlock;
        };
        std::vector<V7Batch> batches;
        v7_build_sync(src, h->sync_cursor, plan, stale_used, batches);
        if (!v7_run_sync(path, batches, err)) { unbind(); return fail(h, TV_ERR_IO, err); }
        h->sync_cursor.gen += 1;
        h->sync_cursor.n_synced = h->n;
        h->sync_pending.clear();
        h->sync_pending.insert(plan.carried.begin(), plan.carried.end());
        h->sync_fresh.clear();
        return TV_OK;
    }

    // First sync of this path, another path than last time, a refit since the last commit, a file that was
    // replaced, or more removals than one header can carry: the whole index as a fresh container, claimed
    // with a new file identity (io_v7.rs write_full :961-1032).
    V7Parts p;
    rc = gather_parts(h, p);
    if (rc != TV_OK) return rc;
    p.nonce = v7_fresh_nonce();
    std::vector<uint8_t> img;
    v7_write_image(p, img);
    if (!v7_write_file_atomic(path, img.data(), img.size(), err)) { unbind(); return fail(h, TV_ERR_IO, err); }
    h->sync_bound = true;
    h->sync_path = path;
    h->sync_cursor = V7Cursor{0, uint64_t(h->n), h->calib_gen, p.nonce};
    h->sync_pending.clear();
    h->sync_fresh.clear();
    return TV_OK;
}

// The planner of an incremental sync on plain arrays (host only; tests).  Outputs: units written into place,
// slots carried by the new header; returns TV_ERR_UNSUPPORTED when the carried ops exceed one header.
int tv_v7_plan_sync(size_t n_synced, size_t n, const size_t *pending, size_t n_pending, const size_t *fresh, size_t n_fresh,
                    size_t *materialise_out, size_t *n_materialise, size_t *carried_out, size_t *n_carried,
                    size_t *append_from, size_t *append_to) {
    if (!n_materialise || !n_carried || (n_pending && !pending) || (n_fresh && !fresh)) return TV_ERR_INVALID_ARGUMENT;
    V7SyncSource src;
    src.n = n;
    V7Cursor cursor;
    cursor.n_synced = n_synced;
    V7SyncPlan plan;
    const std::unordered_set<size_t> ps(pending, pending + n_pending), fs(fresh, fresh + n_fresh);
    if (!v7_plan_sync(src, cursor, ps, fs, plan)) return TV_ERR_UNSUPPORTED;
    if (plan.materialise.size() > *n_materialise || plan.carried.size() > *n_carried) return TV_ERR_INVALID_ARGUMENT;
    std::copy(plan.materialise.begin(), plan.materialise.end(), materialise_out);
    std::copy(plan.carried.begin(), plan.carried.end(), carried_out);
    *n_materialise = plan.materialise.size();
    *n_carried = plan.carried.size();
    if (append_from) *append_from = plan.append_from;
    if (append_to) *append_to = plan.append_to;
    return TV_OK;
}

// Introspection of the sync binding (tests): bound flag, generation and the sizes of the two dirty sets.
int tv_sync_state(const tv_index *h, int *bound, uint64_t *generation, size_t *n_pending, size_t *n_fresh) {
    if (!h) return TV_ERR_INVALID_ARGUMENT;
    std::shared_lock<std::shared_mutex> lock(const_cast<tv_index *>(h)->mu);
    if (bound) *bound = h->sync_bound ? 1 : 0;
    if (generation) *generation = h->sync_cursor.gen;
    if (n_pending) *n_pending = h->sync_pending.size();
    if (n_fresh) *n_fresh = h->sync_fresh.size();
    return TV_OK;
}

int tv_codebook(tv_index *h, float *boundaries_out, float *centroids_out) {
    if (!h) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    if (h->dim == 0) return fail(h, TV_ERR_DIM_NOT_SET, "dimension is not set yet");
    const Codebook &cb = codebook(h->bits, int(h->dim));
    if (boundaries_out) std::copy(cb.boundaries.begin(), cb.boundaries.end(), boundaries_out);
    if (centroids_out) std::copy(cb.centroids.begin(), cb.centroids.end(), centroids_out);
    return TV_OK;
}

int tv_rotate(tv_index *h, const float *rows, size_t n, size_t dim, float *rotated_out) {
    if (!h || !rows || !rotated_out) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    if (h->dim == 0 || dim != h->dim) return fail(h, TV_ERR_DIM_MISMATCH, "tv_rotate needs rows of the index dimension");
    if (n == 0) return TV_OK;
    TV_CUDA(cudaSetDevice(h->device));
    int rc = ensure_tables(h);
    if (rc != TV_OK) return rc;
    cudaStream_t st = h->stream;
    SearchCtx &c = h->ctx[0];                                  // the lock is exclusive: no search holds it
    const size_t nq_pad = (n + 15) / 16 * 16;
    TV_CUDA(h->d_stage.reserve(n * dim));
    TV_CUDA(c.d_qrot.reserve(n * dim));
    TV_CUDA(c.d_qscale.reserve(nq_pad));
    TV_CUDA(c.d_qbias.reserve(nq_pad));
    TV_CUDA(c.d_luts.reserve(n * size_t((h->ngroups + 3) / 4 * 4) * 32));
    TV_CUDA(cudaMemcpyAsync(h->d_stage.ptr, rows, n * dim * 4, cudaMemcpyHostToDevice, st));
    QueryPrepParams qp{};
    qp.queries = h->d_stage.ptr; qp.nq = int(n); qp.dim = int(dim); qp.bits = h->bits; qp.ngroups = h->ngroups;
    qp.mode = kModeLutMulAdd;
    qp.perm0 = h->d_perm.ptr; qp.perm1 = h->d_perm.ptr + dim; qp.inv_sqrt_block = h->rot.inv_sqrt_block;
    qp.centroids = h->d_codebook.ptr + 16;
    qp.q_rot = c.d_qrot.ptr; qp.qscale = c.d_qscale.ptr; qp.qbias = c.d_qbias.ptr; qp.luts = c.d_luts.ptr;
    qp.lut_pitch = (h->ngroups + 3) / 4 * 4 * 32;
    qp.first_invalid = &h->d_flags->first_invalid;
    TV_CUDA(launch_query_prep(qp, st));
    h->launches++;
    TV_CUDA(cudaMemcpyAsync(rotated_out, c.d_qrot.ptr, n * dim * 4, cudaMemcpyDeviceToHost, st));
    TV_CUDA(cudaStreamSynchronize(st));
    return TV_OK;
}

int tv_set_calibration(tv_index *h, size_t dim, const float *shift, const float *scale) {
    if (!h || !shift || !scale) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    if (h->n != 0) return fail(h, TV_ERR_CALIBRATE_NOT_EMPTY, "calibration can only be set on an empty index");
    int rc = validate_dim_for_add(h, dim);
    if (rc != TV_OK) return rc;
    for (size_t d = 0; d < dim; ++d)
        if (!std::isfinite(shift[d]) || !std::isfinite(scale[d]) || !(scale[d] > 0.f))
            return fail(h, TV_ERR_PARTS_INVALID, "calibration entry " + std::to_string(d) + " is not finite or scale is not positive");
    TV_CUDA(cudaSetDevice(h->device));
    h->dim = dim;
    h->shift.assign(shift, shift + dim);
    h->scale_tq.assign(scale, scale + dim);
    h->calib_gen++;
    rc = ensure_tables(h);
    if (rc != TV_OK) return rc;
    return upload_calibration(h);
}

int tv_calibration(const tv_index *h, float *shift_out, float *scale_out, size_t capacity, int *is_calibrated) {
    if (!h) return TV_ERR_INVALID_ARGUMENT;
    if (is_calibrated) *is_calibrated = h->shift.empty() ? 0 : 1;
    if (h->shift.empty()) return TV_OK;
    if (capacity < h->dim) return TV_ERR_INVALID_ARGUMENT;
    if (shift_out) std::copy(h->shift.begin(), h->shift.end(), shift_out);
    if (scale_out) std::copy(h->scale_tq.begin(), h->scale_tq.end(), scale_out);
    return TV_OK;
}

// TQ+ fit: encode::fit_calibration (encode.rs:470-480) = rotate the unit-normalised sample on the device, select
// the two order statistics per coordinate there too, then map the empirical [p_lo, p_hi] quantiles onto the codebook's outer centroids
// (tqplus_anchor encode.rs:364-369, compute_tqplus_calibration :737-857).  Validation order of lib.rs:2599-2640.
int tv_calibrate(tv_index *h, const float *sample, size_t n, size_t dim) {
    if (!h || (!sample && n)) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(h->mu);
    int rc = validate_dim_for_add(h, dim);
    if (rc != TV_OK) return rc;
    if (n < 2) return fail(h, TV_ERR_CALIBRATE_SAMPLE_TOO_SMALL, "calibration needs at least 2 rows, got " + std::to_string(n));
    for (size_t i = 0; i < n * dim; ++i)
        if (!(std::fabs(sample[i]) < kMaxInputMagnitude)) {
            h->err_vec = i / dim; h->err_coord = i % dim; h->err_value = sample[i];
            return fail(h, TV_ERR_INVALID_INPUT_VALUE, "sample row " + std::to_string(i / dim) + " coordinate " + std::to_string(i % dim) + " is not finite or exceeds 1e16 in magnitude");
        }
    TV_CUDA(cudaSetDevice(h->device));
    const bool was_lazy = h->dim == 0;
    if (was_lazy) h->dim = dim;
    auto undo = [&]() { if (was_lazy) { h->dim = 0; h->tables_ready = false; } };
    rc = ensure_tables(h);
    if (rc != TV_OK) { undo(); return rc; }
    const int V = ingest_vectors_per_pass(int(dim), h->ngroups, h->smem_limit);
    if (V == 0) { undo(); return fail(h, TV_ERR_UNSUPPORTED, "dim too large for the ingest kernel's shared memory"); }

    // The rotated sample stays on the device when it fits (a quarter of the free memory at most) and the two order
    // statistics per coordinate are selected there (quantile.cu); a larger sample comes back to the host chunk by chunk
    // and is selected with std::nth_element.
    size_t free_b = 0, total_b = 0;
    TV_CUDA(cudaMemGetInfo(&free_b, &total_b));
    const bool on_device = n * dim * 4 <= free_b / 4 && n <= 0xffffffffull;
    std::vector<float> rotated(on_device ? 0 : n * dim);
    DeviceArray<float> d_rot;
    const size_t chunk_rows = std::max<size_t>(1, std::min<size_t>(n, (size_t(128) << 20) / (dim * 4)));
    TV_CUDA(h->d_stage.reserve(chunk_rows * dim));
    TV_CUDA(d_rot.reserve((on_device ? n : chunk_rows) * dim));
    h->h_flags->first_invalid = ~0ull;
    TV_CUDA(cudaMemcpyAsync(&h->d_flags->first_invalid, &h->h_flags->first_invalid, 8, cudaMemcpyHostToDevice, h->stream));
    IngestParams p{};
    p.dim = int(dim); p.bits = h->bits; p.ngroups = h->ngroups;
    p.perm0 = h->d_perm.ptr; p.perm1 = h->d_perm.ptr + dim; p.inv_sqrt_block = h->rot.inv_sqrt_block;
    p.boundaries = h->d_codebook.ptr; p.centroids = h->d_codebook.ptr + 16;
    p.first_invalid = &h->d_flags->first_invalid;
    for (size_t done = 0; done < n; done += chunk_rows) {
        const size_t rows = std::min(chunk_rows, n - done);
        TV_CUDA(cudaMemcpyAsync(h->d_stage.ptr, sample + done * dim, rows * dim * 4, cudaMemcpyHostToDevice, h->stream));
        p.x = h->d_stage.ptr; p.n = int64_t(rows); p.slot0 = 0; p.row_base = int64_t(done);
        p.rot_out = on_device ? d_rot.ptr + done * dim : d_rot.ptr;
        TV_CUDA(launch_ingest(p, V, h->stream));
        h->launches++;
        if (!on_device) TV_CUDA(cudaMemcpyAsync(rotated.data() + done * dim, d_rot.ptr, rows * dim * 4, cudaMemcpyDeviceToHost, h->stream));
        TV_CUDA(cudaStreamSynchronize(h->stream));           // the staging buffer is reused by the next chunk
    }

    // anchor: probability mass inside the outermost centroid (encode.rs:364-369)
    const double a = (double(dim) - 1.0) / 2.0;
    float c_outer = 0.f;
    for (float c : h->cb.centroids) c_outer = std::fmax(c_outer, std::fabs(c));
    const double p_hi = beta_cdf(a, a, (double(c_outer) + 1.0) / 2.0), p_lo = 1.0 - p_hi;
    const float qc_lo = -c_outer, qc_span = c_outer - qc_lo;
    const size_t lo_idx = size_t(double(n) * p_lo);
    const size_t hi_idx = std::max(std::min(size_t(double(n) * p_hi), n - 1), lo_idx + 1);
    std::vector<float> shift(dim, 0.f), scale(dim, 1.f), col(on_device ? 0 : n), qe(2 * dim);
    if (on_device) {
        DeviceArray<float> d_q;
        TV_CUDA(d_q.reserve(2 * dim));
        TV_CUDA(launch_quantile_pair(d_rot.ptr, int64_t(n), int(dim), int64_t(lo_idx), int64_t(hi_idx), d_q.ptr, d_q.ptr + dim, h->stream));
        h->launches++;
        TV_CUDA(cudaMemcpyAsync(qe.data(), d_q.ptr, 2 * dim * 4, cudaMemcpyDeviceToHost, h->stream));
        TV_CUDA(cudaStreamSynchronize(h->stream));
    } else {
        for (size_t d = 0; d < dim; ++d) {
            for (size_t i = 0; i < n; ++i) col[i] = rotated[i * dim + d];
            std::nth_element(col.begin(), col.begin() + lo_idx, col.end());
            qe[d] = col[lo_idx];
            std::nth_element(col.begin() + lo_idx + 1, col.begin() + hi_idx, col.end());
            qe[dim + d] = col[hi_idx];
        }
    }
    bool identity = true;
    for (size_t d = 0; d < dim; ++d) {
        const float qe_lo = qe[d], qe_hi = qe[dim + d];
        const float qe_span = qe_hi - qe_lo;
        if (qe_span > 1e-6f) {                                       // encode.rs:846-850
            scale[d] = qc_span / qe_span;
            shift[d] = qc_lo / scale[d] - qe_lo;
        }
        if (shift[d] != 0.f || scale[d] != 1.f) identity = false;
    }
    if (identity) { undo(); return fail(h, TV_ERR_CALIBRATE_DEGENERATE_SAMPLE, "the sample yields the identity calibration (degenerate sample)"); }
    if (h->n > 0) {
        // refit: every stored row is re-encoded under the new pair from its own codes (lib.rs:2697-2700, 2760-2832)
        std::vector<float> pair(3 * dim);
        for (size_t d = 0; d < dim; ++d) { pair[d] = shift[d]; pair[dim + d] = scale[d]; pair[2 * dim + d] = 1.0f / scale[d]; }
        DeviceArray<float> d_new;
        TV_CUDA(d_new.reserve(3 * dim));
        TV_CUDA(cudaMemcpyAsync(d_new.ptr, pair.data(), pair.size() * 4, cudaMemcpyHostToDevice, h->stream));
        ReencodeParams rp{};
        rp.codes = h->d_codes; rp.scales = h->d_scales; rp.n = int64_t(h->n);
        rp.dim = int(dim); rp.bits = h->bits; rp.ngroups = h->ngroups;
        rp.boundaries = h->d_codebook.ptr; rp.centroids = h->d_codebook.ptr + 16;
        if (!h->shift.empty()) { rp.old_shift = h->d_calib.ptr; rp.old_inv = h->d_calib.ptr + 2 * dim; }
        rp.new_shift = d_new.ptr; rp.new_scale = d_new.ptr + dim; rp.new_inv = d_new.ptr + 2 * dim;
        TV_CUDA(launch_reencode(rp, h->stream));
        h->expanded.reset();                       // every stored code changed
        h->launches++;
        TV_CUDA(cudaStreamSynchronize(h->stream));
    }
    h->shift = shift;
    h->scale_tq = scale;
    h->calib_gen++;                            // a refit rewrites every stored code: the next sync compacts
    return upload_calibration(h);
}

}  // extern "C"
