// One handle over several GPUs of one process: tv_multi_*.
//
// The reference scans block ranges on different cores and merges per-range candidates by (score descending, slot
// ascending) (turbovec/src/search.rs:3455-3499, 4285-4298).  Here the ranges live on different devices, each in an
// ordinary single-device index (a positional tv_index), and this file is the host logic around them, written against
// the public C ABI only:
//   * ownership is arithmetic.  Global slots are dealt to the shards round-robin in chunks of `chunk_slots`
//     (global block b = slot / 32, chunk = slot / chunk_slots, owner = chunk % G, local slot =
//     (chunk / G) * chunk_slots + slot % chunk_slots), so appends stay balanced at any length and a swap_remove
//     moves one row between two shards at most;
//   * a search uploads the queries to every device, runs tv_search_device_keys on every shard at the same time
//     (one host thread per shard), brings the nq x k result keys of every shard to the first device and merges them
//     there with tv_merge_keys_device_chunked, which also turns local slots into global ones;
//   * masks are given over global slots and cut into per-shard packed words on the host;
//   * an id-mapped handle keeps the reference's two id tables (tv_idtable_*; id_map.rs:221-272) beside the shards:
//     ids never reach a device.
// The same device may be listed more than once (several shards on one GPU): that is how the single-GPU tests run it.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/turbovec_b200.h"

namespace {
constexpr size_t kBlockSlots = 32;

struct Shard {
    int device = 0;
    tv_index *index = nullptr;
    // search scratch on this shard's device
    float *d_queries = nullptr; size_t q_cap = 0;
    uint64_t *d_keys = nullptr; size_t keys_cap = 0;
    uint64_t *d_mask = nullptr; size_t mask_cap = 0;
    std::vector<uint64_t> mask_words;               // this shard's slots of the call's mask
    int rc = 0;                                     // outcome of the shard's part of a call
    std::string message;
};

template <typename T>
cudaError_t grow(T *&ptr, size_t &cap, size_t n) {
    if (n <= cap) return cudaSuccess;
    if (ptr) cudaFree(ptr);
    ptr = nullptr; cap = 0;
    cudaError_t e = cudaMalloc(&ptr, std::max<size_t>(n, 1) * sizeof(T));
    if (e == cudaSuccess) cap = n;
    return e;
}
}  // namespace

struct tv_multi {
    size_t dim = 0;
    int bits = 0, kind = 0;
    size_t chunk_slots = 0;
    size_t n_total = 0;
    std::vector<Shard> shards;
    tv_idtable *table = nullptr;                    // id-mapped handles only
    std::mutex mu;                                  // one call at a time
    std::string last_error;
    uint64_t err_id = 0;
    // merge scratch on the first shard's device, result staging on the host
    uint64_t *d_all_keys = nullptr; size_t all_cap = 0;
    float *d_scores = nullptr; size_t scores_cap = 0;
    int64_t *d_slots = nullptr; size_t slots_cap = 0;
    std::vector<uint64_t> h_keys;
    std::vector<float> h_scores;
    std::vector<int64_t> h_slots;

    size_t world() const { return shards.size(); }
    size_t owner(size_t slot) const { return (slot / chunk_slots) % world(); }
    size_t to_local(size_t slot) const { return (slot / chunk_slots / world()) * chunk_slots + slot % chunk_slots; }
    // number of global slots < n owned by shard r
    size_t local_len(size_t r, size_t n) const {
        const size_t round = chunk_slots * world();
        const size_t full = n / round, rem = n % round;
        const size_t extra = rem > r * chunk_slots ? std::min(rem - r * chunk_slots, chunk_slots) : 0;
        return full * chunk_slots + extra;
    }
};

namespace {
thread_local std::string g_multi_create_error;

int fail(tv_multi *m, int code, const std::string &msg) {
    if (m) m->last_error = msg; else g_multi_create_error = msg;
    return code;
}
int fail_from_shard(tv_multi *m, const Shard &s, int code) {
    return fail(m, code, std::string(tv_last_error(s.index)));
}

// Drops the last `count` rows of a shard (the rows a failed add appended).
void drop_tail(Shard &s, size_t count) {
    for (size_t i = 0; i < count; ++i) {
        const size_t len = tv_len(s.index);
        if (len == 0) break;
        size_t moved = 0;
        tv_swap_remove(s.index, len - 1, &moved);
    }
}

int add_rows(tv_multi *m, const float *vectors, size_t n, size_t dim) {
    if (n == 0) return TV_OK;
    if (m->dim != 0 && dim != m->dim)
        return fail(m, TV_ERR_DIM_MISMATCH, "vector dim " + std::to_string(dim) + " does not match index dim " + std::to_string(m->dim));
    std::vector<size_t> added(m->world(), 0);
    size_t pos = m->n_total;
    const size_t end = pos + n;
    while (pos < end) {
        const size_t next = std::min(end, (pos / m->chunk_slots + 1) * m->chunk_slots);
        Shard &s = m->shards[m->owner(pos)];
        const size_t off = pos - m->n_total, len = next - pos;
        const int rc = tv_add(s.index, vectors + off * dim, len, dim);
        if (rc != TV_OK) {
            // all or nothing (lib.rs:889-930): the runs already appended to other shards are taken back
            std::string msg = tv_last_error(s.index);
            if (rc == TV_ERR_INVALID_INPUT_VALUE) {
                size_t vec = 0, coord = 0; float value = 0.f; uint64_t id = 0;
                tv_error_detail(s.index, &vec, &coord, &value, &id);
                msg = "vector " + std::to_string(off + vec) + " coordinate " + std::to_string(coord) +
                      " is not finite or exceeds 1e16 in magnitude (value " + std::to_string(value) + ")";
            }
            for (size_t r = 0; r < m->world(); ++r) drop_tail(m->shards[r], added[r]);
            return fail(m, rc, msg);
        }
        added[m->owner(pos)] += len;
        pos = next;
    }
    m->n_total = end;
    if (m->dim == 0) m->dim = dim;
    return TV_OK;
}

int swap_remove(tv_multi *m, size_t slot, size_t *moved_from) {
    if (slot >= m->n_total)
        return fail(m, TV_ERR_SLOT_OUT_OF_RANGE, "index " + std::to_string(slot) + " out of bounds (n_vectors = " + std::to_string(m->n_total) + ")");
    const size_t last = m->n_total - 1;
    Shard &hole = m->shards[m->owner(slot)], &tail = m->shards[m->owner(last)];
    const size_t hole_local = m->to_local(slot), last_local = m->to_local(last);
    int rc;
    if (&hole == &tail) {
        size_t moved = 0;
        rc = tv_swap_remove(hole.index, hole_local, &moved);
        if (rc != TV_OK) return fail_from_shard(m, hole, rc);
    } else {
        // lib.rs:2864-3028 across two shards: the last row's codes and scale move into the hole, then the last row goes
        std::vector<uint8_t> groups(m->dim * size_t(m->bits == 2 ? 2 : 4) / 8);      // byte-groups per row: 3-bit codes use 4-bit fields
        float scale = 0.f;
        rc = tv_get_row(tail.index, last_local, groups.data(), groups.size(), &scale);
        if (rc != TV_OK) return fail_from_shard(m, tail, rc);
        rc = tv_set_row(hole.index, hole_local, groups.data(), groups.size(), scale);
        if (rc != TV_OK) return fail_from_shard(m, hole, rc);
        size_t moved = 0;
        rc = tv_swap_remove(tail.index, last_local, &moved);
        if (rc != TV_OK) return fail_from_shard(m, tail, rc);
    }
    m->n_total = last;
    if (moved_from) *moved_from = last;
    return TV_OK;
}

// One shard's part of a search: queries up, keys down (into m->h_keys at list r).
void search_shard(tv_multi *m, size_t r, const float *queries, size_t nq, size_t k, bool masked) {
    Shard &s = m->shards[r];
    s.rc = TV_OK;
    uint64_t *out = m->h_keys.data() + r * nq * k;
    const size_t n_local = tv_len(s.index);
    if (n_local == 0) { std::fill(out, out + nq * k, TV_EMPTY_KEY); return; }
    auto cuda_fail = [&](cudaError_t e) { s.rc = e == cudaErrorMemoryAllocation ? TV_ERR_OUT_OF_MEMORY : TV_ERR_CUDA; s.message = cudaGetErrorString(e); cudaGetLastError(); };
    cudaError_t e = cudaSetDevice(s.device);
    if (e == cudaSuccess) e = grow(s.d_queries, s.q_cap, nq * m->dim);
    if (e == cudaSuccess) e = grow(s.d_keys, s.keys_cap, nq * k);
    if (e == cudaSuccess && masked) e = grow(s.d_mask, s.mask_cap, s.mask_words.size());
    if (e == cudaSuccess) e = cudaMemcpy(s.d_queries, queries, nq * m->dim * sizeof(float), cudaMemcpyHostToDevice);
    if (e == cudaSuccess && masked) e = cudaMemcpy(s.d_mask, s.mask_words.data(), s.mask_words.size() * 8, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { cuda_fail(e); return; }
    size_t k_eff = 0;
    s.rc = tv_search_device_keys(s.index, s.d_queries, nq, k, masked ? s.d_mask : nullptr, 0, s.d_keys, &k_eff);
    if (s.rc != TV_OK) { s.message = tv_last_error(s.index); return; }
    e = cudaMemcpy(out, s.d_keys, nq * k * 8, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) cuda_fail(e);
}

// mask_bool: nullptr or n_total flags over global slots.  Results: rows of *k_eff (scores, global slots).
int search_core(tv_multi *m, const float *queries, size_t nq, size_t dim, size_t k, const uint8_t *mask_bool, std::vector<float> &scores,
                std::vector<int64_t> &slots, size_t *k_eff) {
    *k_eff = 0;
    if (m->n_total == 0 || nq == 0) return TV_OK;                       // lib.rs:1355-1402: an empty index answers with empty rows
    if (dim != m->dim)
        return fail(m, TV_ERR_DIM_MISMATCH, "query dim " + std::to_string(dim) + " does not match index dim " + std::to_string(m->dim));
    const size_t world = m->world();
    size_t kk = std::min(k, m->n_total);
    const bool masked = mask_bool != nullptr;
    if (masked) {
        // cut the global mask into each shard's packed words: whole chunks are runs of chunk_slots / 64 words
        size_t n_allowed = 0;
        for (size_t r = 0; r < world; ++r) m->shards[r].mask_words.assign((m->local_len(r, m->n_total) + 63) / 64, 0);
        for (size_t g = 0; g < m->n_total; ++g) {
            if (!mask_bool[g]) continue;
            ++n_allowed;
            const size_t l = m->to_local(g);
            m->shards[m->owner(g)].mask_words[l >> 6] |= uint64_t(1) << (l & 63);
        }
        kk = std::min(kk, n_allowed);                                       // search.rs:3222-3229
    }
    if (kk == 0) return TV_OK;
    if (world * kk > 8192)
        return fail(m, TV_ERR_UNSUPPORTED, "shards x k = " + std::to_string(world * kk) + " exceeds the merge's 8192 keys per query");
    m->h_keys.resize(world * nq * kk);
    std::vector<std::thread> workers;
    for (size_t r = 1; r < world; ++r) workers.emplace_back(search_shard, m, r, queries, nq, kk, masked);
    search_shard(m, 0, queries, nq, kk, masked);
    for (auto &w : workers) w.join();
    for (size_t r = 0; r < world; ++r)
        if (m->shards[r].rc != TV_OK) return fail(m, m->shards[r].rc, m->shards[r].message);

    const int dev0 = m->shards[0].device;
    cudaError_t e = cudaSetDevice(dev0);
    if (e == cudaSuccess) e = grow(m->d_all_keys, m->all_cap, world * nq * kk);
    if (e == cudaSuccess) e = grow(m->d_scores, m->scores_cap, nq * kk);
    if (e == cudaSuccess) e = grow(m->d_slots, m->slots_cap, nq * kk);
    if (e == cudaSuccess) e = cudaMemcpy(m->d_all_keys, m->h_keys.data(), world * nq * kk * 8, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { cudaGetLastError(); return fail(m, e == cudaErrorMemoryAllocation ? TV_ERR_OUT_OF_MEMORY : TV_ERR_CUDA, cudaGetErrorString(e)); }
    int rc = tv_merge_keys_device_chunked(dev0, m->d_all_keys, world, nq, kk, m->chunk_slots, m->d_scores, m->d_slots, nullptr);
    if (rc != TV_OK) return fail(m, rc, std::string(tv_last_error(nullptr)));
    scores.resize(nq * kk);
    slots.resize(nq * kk);
    e = cudaMemcpy(scores.data(), m->d_scores, nq * kk * sizeof(float), cudaMemcpyDeviceToHost);      // synchronises with the merge
    if (e == cudaSuccess) e = cudaMemcpy(slots.data(), m->d_slots, nq * kk * sizeof(int64_t), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) { cudaGetLastError(); return fail(m, TV_ERR_CUDA, cudaGetErrorString(e)); }
    *k_eff = kk;
    return TV_OK;
}
}  // namespace

extern "C" {

int tv_multi_create(size_t dim, int bit_width, int kind, const int *device_ids, int n_devices, size_t chunk_blocks, tv_multi **out) {
    if (!out) return TV_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    if (!device_ids || n_devices < 1 || n_devices > 64) return fail(nullptr, TV_ERR_INVALID_ARGUMENT, "between 1 and 64 devices are needed");
    if (kind != TV_KIND_POSITIONAL && kind != TV_KIND_IDMAP) return fail(nullptr, TV_ERR_INVALID_ARGUMENT, "unknown index kind");
    if (chunk_blocks == 0) chunk_blocks = 1024;
    if (chunk_blocks % 2) return fail(nullptr, TV_ERR_INVALID_ARGUMENT, "chunk_blocks must be even (chunks are whole 64-bit mask words)");
    tv_multi *m = new tv_multi();
    m->dim = dim; m->bits = bit_width; m->kind = kind;
    m->chunk_slots = chunk_blocks * kBlockSlots;
    m->shards.resize(size_t(n_devices));
    for (int i = 0; i < n_devices; ++i) {
        m->shards[size_t(i)].device = device_ids[i];
        const int rc = tv_index_create(dim, bit_width, TV_KIND_POSITIONAL, device_ids[i], &m->shards[size_t(i)].index);
        if (rc != TV_OK) {
            g_multi_create_error = tv_last_error(nullptr);
            tv_multi_destroy(m);
            return rc;
        }
    }
    if (kind == TV_KIND_IDMAP && tv_idtable_create(&m->table) != TV_OK) {
        tv_multi_destroy(m);
        return fail(nullptr, TV_ERR_OUT_OF_MEMORY, "the id tables could not be created");
    }
    *out = m;
    return TV_OK;
}

void tv_multi_destroy(tv_multi *m) {
    if (!m) return;
    for (Shard &s : m->shards) {
        if (s.d_queries || s.d_keys || s.d_mask) cudaSetDevice(s.device);
        if (s.d_queries) cudaFree(s.d_queries);
        if (s.d_keys) cudaFree(s.d_keys);
        if (s.d_mask) cudaFree(s.d_mask);
        if (s.index) tv_index_destroy(s.index);
    }
    if (m->d_all_keys || m->d_scores || m->d_slots) cudaSetDevice(m->shards[0].device);
    if (m->d_all_keys) cudaFree(m->d_all_keys);
    if (m->d_scores) cudaFree(m->d_scores);
    if (m->d_slots) cudaFree(m->d_slots);
    if (m->table) tv_idtable_destroy(m->table);
    delete m;
}

const char *tv_multi_last_error(const tv_multi *m) { return m ? m->last_error.c_str() : g_multi_create_error.c_str(); }
uint64_t tv_multi_error_id(const tv_multi *m) { return m ? m->err_id : 0; }

size_t tv_multi_len(const tv_multi *mc) {
    tv_multi *m = const_cast<tv_multi *>(mc);
    if (!m) return 0;
    std::lock_guard<std::mutex> lock(m->mu);
    return m->n_total;
}
int tv_multi_shards(const tv_multi *m) { return m ? int(m->shards.size()) : 0; }
tv_index *tv_multi_shard(tv_multi *m, int i) { return m && i >= 0 && size_t(i) < m->shards.size() ? m->shards[size_t(i)].index : nullptr; }

int tv_multi_add(tv_multi *m, const float *vectors, size_t n, size_t dim) {
    if (!m || (!vectors && n)) return TV_ERR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(m->mu);
    if (m->kind != TV_KIND_POSITIONAL) return fail(m, TV_ERR_WRONG_INDEX_KIND, "tv_multi_add on an id-mapped index; use tv_multi_add_with_ids");
    return add_rows(m, vectors, n, dim);
}

int tv_multi_add_with_ids(tv_multi *m, const float *vectors, size_t n, size_t dim, const uint64_t *ids) {
    if (!m || (n && (!vectors || !ids))) return TV_ERR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(m->mu);
    if (m->kind != TV_KIND_IDMAP) return fail(m, TV_ERR_WRONG_INDEX_KIND, "tv_multi_add_with_ids needs an id-mapped index");
    const size_t before = tv_idtable_len(m->table);
    int rc = tv_idtable_add(m->table, ids, n);                          // id checks first, nothing changes on error (id_map.rs:396-434)
    if (rc != TV_OK) { uint64_t id = 0; const char *msg = tv_idtable_last_error(m->table, &id); m->err_id = id; return fail(m, rc, msg); }
    rc = add_rows(m, vectors, n, dim);
    if (rc != TV_OK) tv_idtable_truncate(m->table, before);
    return rc;
}

int tv_multi_swap_remove(tv_multi *m, size_t slot, size_t *moved_from) {
    if (!m) return TV_ERR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(m->mu);
    if (m->kind != TV_KIND_POSITIONAL) return fail(m, TV_ERR_WRONG_INDEX_KIND, "tv_multi_swap_remove on an id-mapped index; use tv_multi_remove");
    return swap_remove(m, slot, moved_from);
}

int tv_multi_remove(tv_multi *m, uint64_t id, int *removed) {
    if (!m) return TV_ERR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(m->mu);
    if (removed) *removed = 0;
    if (m->kind != TV_KIND_IDMAP) return fail(m, TV_ERR_WRONG_INDEX_KIND, "tv_multi_remove needs an id-mapped index");
    int present = 0;
    tv_idtable_contains(m->table, id, &present);
    if (!present) return TV_OK;                                         // id_map.rs:521-523
    // the row first: if moving it fails the tables still describe the index
    uint64_t slot = 0;
    int rc = tv_idtable_resolve(m->table, &id, 1, &slot);
    if (rc != TV_OK) return fail(m, rc, tv_idtable_last_error(m->table, nullptr));
    size_t moved = 0;
    rc = swap_remove(m, size_t(slot), &moved);
    if (rc != TV_OK) return rc;
    int gone = 0; uint64_t s2 = 0, moved2 = 0;
    tv_idtable_remove(m->table, id, &gone, &s2, &moved2);
    if (removed) *removed = gone;
    return TV_OK;
}

int tv_multi_contains(const tv_multi *mc, uint64_t id, int *present) {
    tv_multi *m = const_cast<tv_multi *>(mc);
    if (!m || !present) return TV_ERR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(m->mu);
    *present = 0;
    if (m->kind != TV_KIND_IDMAP) return fail(m, TV_ERR_WRONG_INDEX_KIND, "tv_multi_contains needs an id-mapped index");
    return tv_idtable_contains(m->table, id, present);
}

int tv_multi_ids(const tv_multi *mc, uint64_t *ids_out, size_t capacity) {
    tv_multi *m = const_cast<tv_multi *>(mc);
    if (!m || (!ids_out && capacity)) return TV_ERR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(m->mu);
    if (m->kind != TV_KIND_IDMAP) return fail(m, TV_ERR_WRONG_INDEX_KIND, "tv_multi_ids needs an id-mapped index");
    return tv_idtable_ids(m->table, ids_out, capacity);
}

int tv_multi_search(tv_multi *m, const float *queries, size_t nq, size_t dim, size_t k, const uint8_t *mask_bool, size_t mask_len,
                    float *scores_out, int64_t *slots_out, size_t *k_eff) {
    if (!m || !k_eff || (!queries && nq)) return TV_ERR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(m->mu);
    if (m->kind != TV_KIND_POSITIONAL) return fail(m, TV_ERR_WRONG_INDEX_KIND, "tv_multi_search on an id-mapped index; use tv_multi_search_allowlist");
    if (mask_bool && mask_len != m->n_total)                             // lib.rs:1427-1433
        return fail(m, TV_ERR_MASK_LENGTH_MISMATCH, "mask length " + std::to_string(mask_len) + " does not match index size " + std::to_string(m->n_total));
    int rc = search_core(m, queries, nq, dim, k, mask_bool, m->h_scores, m->h_slots, k_eff);
    if (rc != TV_OK || *k_eff == 0) return rc;
    if (scores_out) std::copy(m->h_scores.begin(), m->h_scores.begin() + nq * *k_eff, scores_out);
    if (slots_out) std::copy(m->h_slots.begin(), m->h_slots.begin() + nq * *k_eff, slots_out);
    return TV_OK;
}

int tv_multi_search_allowlist(tv_multi *m, const float *queries, size_t nq, size_t dim, size_t k, const uint64_t *allow_ids, size_t n_allow,
                              float *scores_out, uint64_t *ids_out, size_t *k_eff) {
    if (!m || !k_eff || (!queries && nq)) return TV_ERR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(m->mu);
    if (m->kind != TV_KIND_IDMAP) return fail(m, TV_ERR_WRONG_INDEX_KIND, "tv_multi_search_allowlist needs an id-mapped index");
    std::vector<uint8_t> mask;
    if (allow_ids) {                                                    // id_map.rs:670-683
        std::vector<uint64_t> slots(n_allow);
        int rc = tv_idtable_resolve(m->table, allow_ids, n_allow, slots.data());
        if (rc != TV_OK) { uint64_t id = 0; const char *msg = tv_idtable_last_error(m->table, &id); m->err_id = id; return fail(m, rc, msg); }
        mask.assign(m->n_total, 0);
        for (uint64_t s : slots) mask[size_t(s)] = 1;
    }
    int rc = search_core(m, queries, nq, dim, k, allow_ids ? mask.data() : nullptr, m->h_scores, m->h_slots, k_eff);
    if (rc != TV_OK || *k_eff == 0) return rc;
    if (scores_out) std::copy(m->h_scores.begin(), m->h_scores.begin() + nq * *k_eff, scores_out);
    if (ids_out) {                                                      // id_map.rs:695-705
        rc = tv_idtable_ids_of(m->table, m->h_slots.data(), nq * *k_eff, ids_out);
        if (rc != TV_OK) return fail(m, rc, tv_idtable_last_error(m->table, nullptr));
    }
    return TV_OK;
}

}  // extern "C"
