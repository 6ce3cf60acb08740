// Test-only stand-in for the single-device index behind csrc/multi.cpp: the subset of the C ABI that file calls,
// implemented by brute force on the host.  A row is stored as dim / 2 code bytes (two 4-bit codes per byte, a crude
// uniform quantiser) plus a scale, so that tv_get_row / tv_set_row move exactly what the real index moves; a score
// is scale * sum_d q[d] * (code_d - 8), accumulated in double and rounded once.  Keys use an order-preserving image
// of the score so that ascending key order = (score descending, slot ascending), as the real library's do.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/turbovec_b200.h"

struct tv_index {
    size_t dim = 0;
    int bits = 4;
    std::vector<std::vector<uint8_t>> codes;
    std::vector<float> scales;
    std::string last_error;
    size_t err_vec = 0, err_coord = 0;
    float err_value = 0.f;
};

namespace {
thread_local std::string g_error;
int fail(tv_index *h, int code, const std::string &msg) { if (h) h->last_error = msg; else g_error = msg; return code; }
uint32_t desc_bits(float s) {
    uint32_t u; std::memcpy(&u, &s, 4);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);           // ascending with the score
    return ~u;                                                 // descending
}
float score_of_bits(uint32_t d) {
    uint32_t u = ~d;
    u = (u & 0x80000000u) ? (u & 0x7fffffffu) : ~u;
    float s; std::memcpy(&s, &u, 4); return s;
}
}  // namespace

extern "C" {

int tv_index_create(size_t dim, int bit_width, int kind, int, tv_index **out) {
    if (bit_width != 4 || kind != TV_KIND_POSITIONAL || dim % 8) return fail(nullptr, TV_ERR_INVALID_ARGUMENT, "fake index: 4-bit positional only");
    *out = new tv_index();
    (*out)->dim = dim;
    return TV_OK;
}
void tv_index_destroy(tv_index *h) { delete h; }
const char *tv_last_error(const tv_index *h) { return h ? h->last_error.c_str() : g_error.c_str(); }
void tv_error_detail(const tv_index *h, size_t *v, size_t *c, float *value, uint64_t *id) {
    if (v) *v = h->err_vec; if (c) *c = h->err_coord; if (value) *value = h->err_value; if (id) *id = 0;
}
size_t tv_len(const tv_index *h) { return h ? h->codes.size() : 0; }

int tv_add(tv_index *h, const float *x, size_t n, size_t dim) {
    if (h->dim == 0) h->dim = dim;
    if (dim != h->dim) return fail(h, TV_ERR_DIM_MISMATCH, "dim mismatch");
    for (size_t i = 0; i < n * dim; ++i)
        if (!(std::fabs(x[i]) < 1e16f)) { h->err_vec = i / dim; h->err_coord = i % dim; h->err_value = x[i]; return fail(h, TV_ERR_INVALID_INPUT_VALUE, "invalid value"); }
    for (size_t r = 0; r < n; ++r) {
        const float *row = x + r * dim;
        double norm = 0; for (size_t d = 0; d < dim; ++d) norm += double(row[d]) * row[d];
        norm = std::sqrt(norm);
        std::vector<uint8_t> c(dim / 2);
        for (size_t g = 0; g < dim / 2; ++g) {
            auto q = [&](float v) { int k = int(std::lround((norm > 0 ? v / norm : 0.0) * 24.0)) + 8; return uint8_t(std::min(15, std::max(0, k))); };
            c[g] = uint8_t(q(row[2 * g]) << 4 | q(row[2 * g + 1]));
        }
        h->codes.push_back(c);
        h->scales.push_back(float(norm / 24.0));
    }
    return TV_OK;
}
int tv_swap_remove(tv_index *h, size_t slot, size_t *moved_from) {
    if (slot >= h->codes.size()) return fail(h, TV_ERR_SLOT_OUT_OF_RANGE, "slot out of range");
    const size_t last = h->codes.size() - 1;
    h->codes[slot] = h->codes[last]; h->scales[slot] = h->scales[last];
    h->codes.pop_back(); h->scales.pop_back();
    if (moved_from) *moved_from = last;
    return TV_OK;
}
int tv_get_row(const tv_index *h, size_t slot, uint8_t *groups, size_t capacity, float *scale) {
    if (slot >= h->codes.size() || capacity < h->dim / 2) return TV_ERR_INVALID_ARGUMENT;
    std::copy(h->codes[slot].begin(), h->codes[slot].end(), groups);
    *scale = h->scales[slot];
    return TV_OK;
}
int tv_set_row(tv_index *h, size_t slot, const uint8_t *groups, size_t count, float scale) {
    if (slot >= h->codes.size() || count != h->dim / 2) return TV_ERR_INVALID_ARGUMENT;
    h->codes[slot].assign(groups, groups + count);
    h->scales[slot] = scale;
    return TV_OK;
}
int tv_search_device_keys(tv_index *h, const float *q, size_t nq, size_t k, const uint64_t *mask, uint64_t slot_offset, uint64_t *keys, size_t *k_eff) {
    const size_t n = h->codes.size(), dim = h->dim;
    size_t best = 0;
    for (size_t i = 0; i < nq; ++i) {
        std::vector<uint64_t> all;
        for (size_t s = 0; s < n; ++s) {
            if (mask && !((mask[s >> 6] >> (s & 63)) & 1)) continue;
            double acc = 0;
            for (size_t g = 0; g < dim / 2; ++g)
                acc += double(q[i * dim + 2 * g]) * (int(h->codes[s][g] >> 4) - 8) + double(q[i * dim + 2 * g + 1]) * (int(h->codes[s][g] & 15) - 8);
            const float score = float(acc * h->scales[s]);
            all.push_back(uint64_t(desc_bits(score)) << 32 | uint64_t(s + slot_offset));
        }
        std::sort(all.begin(), all.end());
        for (size_t j = 0; j < k; ++j) keys[i * k + j] = j < all.size() ? all[j] : TV_EMPTY_KEY;
        best = std::max(best, std::min(k, all.size()));
    }
    if (k_eff) *k_eff = best;
    return TV_OK;
}
int tv_merge_keys_device_chunked(int, const uint64_t *keys, size_t n_lists, size_t nq, size_t k, size_t chunk_slots, float *scores, int64_t *slots, void *) {
    for (size_t i = 0; i < nq; ++i) {
        std::vector<uint64_t> all;
        for (size_t r = 0; r < n_lists; ++r)
            for (size_t j = 0; j < k; ++j) {
                const uint64_t key = keys[(r * nq + i) * k + j];
                if (key == TV_EMPTY_KEY) continue;
                const uint64_t local = key & 0xffffffffull;
                const uint64_t global = ((local / chunk_slots) * n_lists + r) * chunk_slots + local % chunk_slots;
                all.push_back((key & 0xffffffff00000000ull) | global);
            }
        std::sort(all.begin(), all.end());
        for (size_t j = 0; j < k; ++j) {
            const bool have = j < all.size();
            scores[i * k + j] = have ? score_of_bits(uint32_t(all[j] >> 32)) : -INFINITY;
            slots[i * k + j] = have ? int64_t(all[j] & 0xffffffffull) : 0;
        }
    }
    return TV_OK;
}

}  // extern "C"
