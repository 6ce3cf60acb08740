// Stand-alone id <-> slot tables: what IdMapIndex keeps around its inner index in the reference
// (turbovec/src/id_map.rs:221-272: slot_to_id plus the id_to_slot map), without any vectors.
//
// A slot-sharded index (one process per GPU) numbers slots globally, so the id tables are global state: every rank
// keeps a replica and applies the same operations in the same order.  The tables never touch the device.
#include <algorithm>
#include <cstdint>
#include <mutex>
#include <shared_mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../../include/turbovec_b200.h"

struct tv_idtable {
    std::vector<uint64_t> slot_to_id;
    std::unordered_map<uint64_t, uint64_t> id_to_slot;
    mutable std::shared_mutex mu;
    mutable std::mutex err_mu;
    mutable std::string last_error;
    mutable uint64_t err_id = 0;
};

namespace {
int fail(const tv_idtable *t, int code, uint64_t id, const std::string &msg) {
    std::lock_guard<std::mutex> g(t->err_mu);
    t->last_error = msg;
    t->err_id = id;
    return code;
}
}  // namespace

extern "C" {

int tv_idtable_create(tv_idtable **out) {
    if (!out) return TV_ERR_INVALID_ARGUMENT;
    *out = new tv_idtable();
    return TV_OK;
}

void tv_idtable_destroy(tv_idtable *t) { delete t; }

size_t tv_idtable_len(const tv_idtable *t) {
    if (!t) return 0;
    std::shared_lock<std::shared_mutex> lock(t->mu);
    return t->slot_to_id.size();
}

const char *tv_idtable_last_error(const tv_idtable *t, uint64_t *id) {
    if (!t) return "";
    std::lock_guard<std::mutex> g(t->err_mu);
    if (id) *id = t->err_id;
    return t->last_error.c_str();
}

// add_with_ids_2d's id checks, per id and in order: already present, then duplicate within the batch
// (id_map.rs:396-434); nothing changes on error.  The new ids take the slots len .. len + n - 1.
int tv_idtable_add(tv_idtable *t, const uint64_t *ids, size_t n) {
    if (!t || (!ids && n)) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(t->mu);
    std::unordered_set<uint64_t> seen;
    seen.reserve(n * 2);
    for (size_t i = 0; i < n; ++i) {
        if (t->id_to_slot.count(ids[i])) return fail(t, TV_ERR_ID_ALREADY_PRESENT, ids[i], "id " + std::to_string(ids[i]) + " is already present");
        if (!seen.insert(ids[i]).second) return fail(t, TV_ERR_DUPLICATE_ID_IN_BATCH, ids[i], "id " + std::to_string(ids[i]) + " appears twice in the batch");
    }
    const uint64_t base = t->slot_to_id.size();
    t->slot_to_id.insert(t->slot_to_id.end(), ids, ids + n);
    t->id_to_slot.reserve(t->id_to_slot.size() + n);
    for (size_t i = 0; i < n; ++i) t->id_to_slot.emplace(ids[i], base + i);
    return TV_OK;
}

// Drops the slots n .. len - 1 again (undo of an add whose vectors were then rejected).
int tv_idtable_truncate(tv_idtable *t, size_t n) {
    if (!t) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(t->mu);
    while (t->slot_to_id.size() > n) {
        t->id_to_slot.erase(t->slot_to_id.back());
        t->slot_to_id.pop_back();
    }
    return TV_OK;
}

// IdMapIndex::remove's table update (id_map.rs:520-567): the last slot's id moves into the freed slot.
// *slot = the freed slot, *moved_from = the slot whose row takes its place (the last one; equal to *slot when the
// removed id held the last slot).  An unknown id is not an error: *removed = 0.
int tv_idtable_remove(tv_idtable *t, uint64_t id, int *removed, uint64_t *slot, uint64_t *moved_from) {
    if (!t) return TV_ERR_INVALID_ARGUMENT;
    std::unique_lock<std::shared_mutex> lock(t->mu);
    if (removed) *removed = 0;
    auto it = t->id_to_slot.find(id);
    if (it == t->id_to_slot.end()) return TV_OK;
    const uint64_t s = it->second, last = t->slot_to_id.size() - 1;
    t->id_to_slot.erase(it);
    if (s != last) {
        const uint64_t moved = t->slot_to_id[last];
        t->slot_to_id[s] = moved;
        t->id_to_slot[moved] = s;
    }
    t->slot_to_id.pop_back();
    if (removed) *removed = 1;
    if (slot) *slot = s;
    if (moved_from) *moved_from = last;
    return TV_OK;
}

int tv_idtable_contains(const tv_idtable *t, uint64_t id, int *present) {
    if (!t || !present) return TV_ERR_INVALID_ARGUMENT;
    std::shared_lock<std::shared_mutex> lock(t->mu);
    *present = t->id_to_slot.count(id) ? 1 : 0;
    return TV_OK;
}

// Allowlist ids -> global slots (id_map.rs:670-683): an empty list and an unknown id are errors; the unknown id
// reported is the first one in list order.  Large lists are split over host threads (the lookups only read).
int tv_idtable_resolve(const tv_idtable *t, const uint64_t *ids, size_t n, uint64_t *slots_out) {
    if (!t || (!ids && n) || (!slots_out && n)) return TV_ERR_INVALID_ARGUMENT;
    std::shared_lock<std::shared_mutex> lock(t->mu);
    if (n == 0) return fail(t, TV_ERR_ALLOWLIST_EMPTY, 0, "allowlist is empty");
    const size_t n_threads = n < (size_t(1) << 16) ? 1 : std::min<size_t>(16, std::max(1u, std::thread::hardware_concurrency()));
    std::vector<size_t> first_unknown(n_threads, n);
    auto work = [&](size_t th) {
        const size_t lo = n * th / n_threads, hi = n * (th + 1) / n_threads;
        for (size_t i = lo; i < hi; ++i) {
            auto it = t->id_to_slot.find(ids[i]);
            if (it == t->id_to_slot.end()) { first_unknown[th] = i; return; }
            slots_out[i] = it->second;
        }
    };
    if (n_threads == 1) {
        work(0);
    } else {
        std::vector<std::thread> pool;
        for (size_t th = 0; th < n_threads; ++th) pool.emplace_back(work, th);
        for (auto &p : pool) p.join();
    }
    const size_t bad = *std::min_element(first_unknown.begin(), first_unknown.end());
    if (bad < n) return fail(t, TV_ERR_UNKNOWN_ID, ids[bad], "allowlist id " + std::to_string(ids[bad]) + " is not in the index");
    return TV_OK;
}

// slots -> ids (id_map.rs:695-705); slots must be below len.
int tv_idtable_ids_of(const tv_idtable *t, const int64_t *slots, size_t n, uint64_t *ids_out) {
    if (!t || (!slots && n) || (!ids_out && n)) return TV_ERR_INVALID_ARGUMENT;
    std::shared_lock<std::shared_mutex> lock(t->mu);
    const size_t len = t->slot_to_id.size();
    for (size_t i = 0; i < n; ++i) {
        if (slots[i] < 0 || size_t(slots[i]) >= len) return fail(t, TV_ERR_SLOT_OUT_OF_RANGE, 0, "slot " + std::to_string(slots[i]) + " out of range");
        ids_out[i] = t->slot_to_id[size_t(slots[i])];
    }
    return TV_OK;
}

int tv_idtable_ids(const tv_idtable *t, uint64_t *ids_out, size_t capacity) {
    if (!t || (!ids_out && capacity)) return TV_ERR_INVALID_ARGUMENT;
    std::shared_lock<std::shared_mutex> lock(t->mu);
    if (capacity < t->slot_to_id.size()) return TV_ERR_INVALID_ARGUMENT;
    std::copy(t->slot_to_id.begin(), t->slot_to_id.end(), ids_out);
    return TV_OK;
}

}  // extern "C"
