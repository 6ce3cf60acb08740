#include "io_v7.hpp"

#include <algorithm>
#include <cerrno>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

namespace tv {
namespace {

constexpr size_t kBlk = 32;
constexpr size_t kMaxOps = 1024;          // io_v7.rs MAX_OPS
constexpr uint8_t kMagic[4] = {'T', 'V', '7', 0};
constexpr uint8_t kRevision = 2;

struct Crc32cTable {
    uint32_t t[256];
    Crc32cTable() {
        for (uint32_t i = 0; i < 256; ++i) {
            uint32_t c = i;
            for (int k = 0; k < 8; ++k) c = (c & 1) ? (c >> 1) ^ 0x82F63B78u : c >> 1;   // Castagnoli, reflected
            t[i] = c;
        }
    }
};
uint32_t crc_update(uint32_t crc, const uint8_t *d, size_t n) {
    static const Crc32cTable table;
    for (size_t i = 0; i < n; ++i) crc = table.t[(crc ^ d[i]) & 0xff] ^ (crc >> 8);
    return crc;
}
uint32_t crc_one(const uint8_t *d, size_t n) { return ~crc_update(0xFFFFFFFFu, d, n); }

// The delta digest over pieces that are not contiguous: same split points as crc32c_split on the
// concatenation (io_v7.rs:276-345).
struct PieceDigest {
    size_t at = 0, s1 = 0, s2 = 0;
    bool split;
    uint32_t part[3] = {0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu};
    explicit PieceDigest(size_t total) : split(total >= 4096) {
        if (split) { s1 = total / 3; s2 = s1 * 2; }
    }
    void push(const uint8_t *d, size_t n) {
        if (!split) { part[0] = crc_update(part[0], d, n); at += n; return; }
        while (n) {
            const int which = at < s1 ? 0 : (at < s2 ? 1 : 2);
            const size_t end = which == 0 ? s1 : (which == 1 ? s2 : SIZE_MAX);
            const size_t take = n < end - at ? n : end - at;
            part[which] = crc_update(part[which], d, take);
            at += take; d += take; n -= take;
        }
    }
    uint32_t finish() const {
        if (!split) return ~part[0];
        uint8_t digest[12];
        for (int i = 0; i < 3; ++i) { const uint32_t v = ~part[i]; std::memcpy(digest + 4 * i, &v, 4); }
        return crc_one(digest, 12);
    }
};

struct Geo {
    int kind, bits;
    size_t dim, n_calib;
    size_t row_bytes() const { return dim / size_t(8 / bits); }
    size_t levels() const { return size_t(1) << bits; }
    size_t id_bytes(size_t rows) const { return kind == 1 ? rows * 8 : 0; }
    size_t sb_len() const { return 23 + (levels() - 1) * 4 + levels() * 4 + 4 + n_calib * 8 + 4; }
    size_t op_size() const { return 1 + row_bytes() + 4 + id_bytes(1); }
    size_t hdr_len() const {
        return 16 + 31 * (row_bytes() + 4 + id_bytes(1)) + 4 + kMaxOps * (5 + op_size()) + 4 + kMaxOps * 4 + 12 + 4;
    }
    size_t hdr_at(size_t slot) const { return sb_len() + slot * hdr_len(); }
    size_t unit_len() const { return kBlk * row_bytes() + kBlk * 4 + id_bytes(kBlk); }
    size_t unit_at(size_t block) const { return hdr_at(2) + block * unit_len(); }
};

template <typename T>
void put(std::vector<uint8_t> &v, T x) {
    uint8_t b[sizeof(T)];
    std::memcpy(b, &x, sizeof(T));
    v.insert(v.end(), b, b + sizeof(T));
}
template <typename T>
bool get(const uint8_t *d, size_t len, size_t at, T &x) {
    if (at + sizeof(T) > len) return false;
    std::memcpy(&x, d + at, sizeof(T));
    return true;
}

// One row's byte-groups in group order out of the blocked array.
void row_codes(const std::vector<uint8_t> &blocked, size_t rb, size_t r, uint8_t *out) {
    const uint8_t *base = blocked.data() + (r / kBlk) * rb * kBlk + (r % kBlk);
    for (size_t g = 0; g < rb; ++g) out[g] = base[g * kBlk];
}

}  // namespace

uint32_t crc32c_split(const uint8_t *data, size_t len) {
    if (len < 4096) return crc_one(data, len);
    const size_t third = len / 3;
    const uint32_t parts[3] = {crc_one(data, third), crc_one(data + third, third), crc_one(data + 2 * third, len - 2 * third)};
    uint8_t digest[12];
    std::memcpy(digest, parts, 12);
    return crc_one(digest, 12);
}

size_t v7_image_len(const V7Parts &p) {
    const Geo g{p.kind, p.bits, p.dim, p.shift.size()};
    return g.unit_at(p.n / kBlk);
}

void v7_write_image(const V7Parts &p, std::vector<uint8_t> &out) {
    const Geo g{p.kind, p.bits, p.dim, p.shift.size()};
    const size_t rb = p.dim ? g.row_bytes() : 0;
    out.clear();
    out.reserve(g.unit_at(p.n / kBlk));
    // superblock
    out.insert(out.end(), kMagic, kMagic + 4);
    out.push_back(kRevision);
    out.push_back(uint8_t(p.bits));
    out.push_back(uint8_t(p.kind));
    put<uint32_t>(out, uint32_t(p.dim));
    put<uint64_t>(out, p.nonce);                             // 0 = unclaimed snapshot
    put<uint32_t>(out, uint32_t(kMaxOps));
    for (float v : p.boundaries) put<float>(out, v);
    for (float v : p.centroids) put<float>(out, v);
    put<uint32_t>(out, uint32_t(p.shift.size()));
    for (float v : p.shift) put<float>(out, v);
    for (float v : p.scale) put<float>(out, v);
    put<uint32_t>(out, crc32c_split(out.data(), out.size()));
    // header slot 0: generation 0, n, tail rows, no op groups, empty delta
    const size_t h0 = out.size();
    put<uint64_t>(out, 0);
    put<uint64_t>(out, uint64_t(p.n));
    const size_t n_tail = p.n % kBlk, first_tail = p.n - n_tail;
    std::vector<uint8_t> row(rb);
    for (size_t k = 0; k < n_tail; ++k) {
        const size_t r = first_tail + k;
        row_codes(p.blocked, rb, r, row.data());
        out.insert(out.end(), row.begin(), row.end());
        put<float>(out, p.scales[r]);
        if (p.kind == 1) put<uint64_t>(out, p.ids[r]);
    }
    put<uint32_t>(out, 0);                                   // op groups
    put<uint32_t>(out, 0);                                   // materialised units
    put<uint32_t>(out, 0);                                   // appended range start
    put<uint32_t>(out, 0);                                   // appended range end
    {
        const uint64_t gen = 0;
        put<uint32_t>(out, crc_one(reinterpret_cast<const uint8_t *>(&gen), 8));   // delta digest of the 8 gen bytes
    }
    put<uint32_t>(out, crc32c_split(out.data() + h0, out.size() - h0));
    out.resize(h0 + 2 * g.hdr_len(), 0);                     // pad slot 0, slot 1 all zero
    // whole-block units
    for (size_t b = 0; b < p.n / kBlk; ++b) {
        out.insert(out.end(), p.blocked.begin() + b * rb * kBlk, p.blocked.begin() + (b + 1) * rb * kBlk);
        for (size_t l = 0; l < kBlk; ++l) put<float>(out, p.scales[b * kBlk + l]);
        if (p.kind == 1)
            for (size_t l = 0; l < kBlk; ++l) put<uint64_t>(out, p.ids[b * kBlk + l]);
    }
}

namespace {
struct ParsedHeader {
    uint64_t gen = 0;
    size_t n = 0, tail_at = 0, used = 0;
    std::vector<std::pair<size_t, size_t>> ops;              // (slot, offset of codes in the file)
    std::vector<size_t> delta_units;
    uint32_t delta_crc = 0;
};

// Structure and checksum of one header slot (io_v7.rs parse_header_at).  `b` points at the slot's bytes, of
// which `cap` are present; `at` is the slot's file offset and `file_len` the length the units must fit in.
bool parse_header_bytes(const uint8_t *b, size_t cap, size_t at, const Geo &g, size_t slot, size_t file_len, ParsedHeader &h) {
    uint64_t gen, n64;
    if (!get(b, cap, 0, gen) || !get(b, cap, 8, n64)) return false;
    if (gen % 2 != slot) return false;
    const size_t n = size_t(n64);
    if (n / kBlk > (SIZE_MAX - g.unit_at(0)) / g.unit_len() || g.unit_at(n / kBlk) > file_len) return false;
    const size_t tail_row = g.row_bytes() + 4 + g.id_bytes(1);
    size_t p = 16 + (n % kBlk) * tail_row;
    uint32_t n_groups;
    if (!get(b, cap, p, n_groups) || n_groups > kMaxOps) return false;
    p += 4;
    h.ops.clear();
    for (uint32_t gi = 0; gi < n_groups; ++gi) {
        uint32_t blk;
        uint8_t n_ops;
        if (!get(b, cap, p, blk) || !get(b, cap, p + 4, n_ops) || blk >= n / kBlk) return false;
        p += 5;
        for (uint8_t o = 0; o < n_ops; ++o) {
            uint8_t lane;
            if (!get(b, cap, p, lane) || lane >= kBlk || p + g.op_size() > cap) return false;
            h.ops.push_back({size_t(blk) * kBlk + lane, at + p + 1});
            p += g.op_size();
        }
    }
    uint32_t n_mat;
    if (!get(b, cap, p, n_mat) || n_mat > kMaxOps) return false;
    p += 4;
    h.delta_units.clear();
    for (uint32_t i = 0; i < n_mat; ++i) {
        uint32_t u;
        if (!get(b, cap, p, u)) return false;
        h.delta_units.push_back(u);
        p += 4;
    }
    uint32_t from, to, stored;
    if (!get(b, cap, p, from) || !get(b, cap, p + 4, to) || !get(b, cap, p + 8, h.delta_crc)) return false;
    p += 12;
    if (!get(b, cap, p, stored) || crc32c_split(b, p) != stored) return false;
    if (to > from && size_t(to - from) > file_len / g.unit_len() + 1) return false;   // cannot all be in the file
    for (uint32_t u = from; u < to; ++u) h.delta_units.push_back(u);
    h.gen = gen; h.n = n; h.tail_at = at + 16; h.used = p + 4;
    return true;
}

// The delta check: the units this commit wrote are in the file as it wrote them (io_v7.rs delta_verified).
// `unit(u)` returns the unit's bytes or null when they are not there.
template <typename F>
bool delta_verified(const ParsedHeader &h, const Geo &g, F &&unit) {
    PieceDigest dg(8 + h.delta_units.size() * (4 + g.unit_len()));
    dg.push(reinterpret_cast<const uint8_t *>(&h.gen), 8);
    for (size_t u : h.delta_units) {
        const uint8_t *bytes = unit(u);
        if (!bytes) return false;
        const uint32_t u32 = uint32_t(u);
        dg.push(reinterpret_cast<const uint8_t *>(&u32), 4);
        dg.push(bytes, g.unit_len());
    }
    return dg.finish() == h.delta_crc;
}

bool parse_header(const uint8_t *d, size_t len, const Geo &g, size_t slot, ParsedHeader &h) {
    const size_t at = g.hdr_at(slot);
    if (at + g.hdr_len() > len) return false;
    if (!parse_header_bytes(d + at, g.hdr_len(), at, g, slot, len, h)) return false;
    return delta_verified(h, g, [&](size_t u) -> const uint8_t * { return g.unit_at(u + 1) <= len ? d + g.unit_at(u) : nullptr; });
}
}  // namespace

bool v7_read_image(const uint8_t *d, size_t len, V7Parts &out, std::string &error) {
    if (len < 11 || std::memcmp(d, kMagic, 4) != 0) { error = "not a v7 file"; return false; }
    if (d[4] != kRevision) { error = "unsupported v7 revision " + std::to_string(int(d[4])); return false; }
    out.bits = d[5];
    if (out.bits < 2 || out.bits > 4) { error = "bit_width " + std::to_string(out.bits) + " out of range"; return false; }
    out.kind = d[6];
    if (out.kind > 1) { error = "unknown v7 index kind " + std::to_string(out.kind); return false; }
    uint32_t dim, max_ops, n_calib;
    if (!get(d, len, 7, dim) || !get(d, len, 19, max_ops)) { error = "truncated superblock"; return false; }
    if (dim != 0 && (dim % 8 != 0 || dim > 16384)) { error = "dim " + std::to_string(dim) + " invalid"; return false; }
    if (max_ops != kMaxOps) { error = "unexpected redo-op capacity " + std::to_string(max_ops); return false; }
    out.dim = dim;
    const size_t levels = size_t(1) << out.bits;
    size_t p = 23;
    out.boundaries.resize(levels - 1);
    out.centroids.resize(levels);
    for (auto &v : out.boundaries) { if (!get(d, len, p, v)) { error = "truncated superblock"; return false; } p += 4; }
    for (auto &v : out.centroids) { if (!get(d, len, p, v)) { error = "truncated superblock"; return false; } p += 4; }
    if (!get(d, len, p, n_calib) || (n_calib != 0 && n_calib != dim)) { error = "calibration length invalid"; return false; }
    p += 4;
    out.shift.resize(n_calib);
    out.scale.resize(n_calib);
    for (auto &v : out.shift) { if (!get(d, len, p, v)) { error = "truncated superblock"; return false; } p += 4; }
    for (auto &v : out.scale) { if (!get(d, len, p, v)) { error = "truncated superblock"; return false; } p += 4; }
    uint32_t stored;
    if (!get(d, len, p, stored) || crc32c_split(d, p) != stored) { error = "superblock checksum mismatch"; return false; }
    for (size_t i = 0; dim != 0 && i + 1 < out.centroids.size(); ++i)   // a lazy index carries a placeholder codebook
        if (!(out.centroids[i] < out.centroids[i + 1])) { error = "codebook centroids are not ascending"; return false; }
    for (size_t i = 0; i < n_calib; ++i)
        if (!std::isfinite(out.shift[i]) || !std::isfinite(out.scale[i]) || !(out.scale[i] > 0.f)) { error = "calibration entry invalid"; return false; }

    const Geo g{out.kind, out.bits, out.dim, n_calib};
    ParsedHeader h[2];
    const bool ok0 = parse_header(d, len, g, 0, h[0]), ok1 = parse_header(d, len, g, 1, h[1]);
    if (!ok0 && !ok1) { error = "no valid commit header"; return false; }
    const ParsedHeader &hd = (ok0 && ok1) ? (h[0].gen > h[1].gen ? h[0] : h[1]) : (ok0 ? h[0] : h[1]);
    const size_t n = hd.n, rb = dim ? g.row_bytes() : 0, n_full = n / kBlk;
    out.n = n;
    out.gen = hd.gen;
    std::memcpy(&out.nonce, d + 11, 8);
    out.pending_slots.clear();
    for (const auto &op : hd.ops) out.pending_slots.push_back(op.first);
    out.blocked.assign(((n + kBlk - 1) / kBlk) * rb * kBlk, 0);
    out.scales.assign(n, 0.f);
    out.ids.assign(out.kind == 1 ? n : 0, 0);
    for (size_t b = 0; b < n_full; ++b) {
        const uint8_t *u = d + g.unit_at(b);
        std::memcpy(out.blocked.data() + b * rb * kBlk, u, rb * kBlk);
        std::memcpy(out.scales.data() + b * kBlk, u + rb * kBlk, kBlk * 4);
        if (out.kind == 1) std::memcpy(out.ids.data() + b * kBlk, u + rb * kBlk + kBlk * 4, kBlk * 8);
    }
    auto place_row = [&](size_t slot, const uint8_t *src) {       // codes | scale | id
        uint8_t *base = out.blocked.data() + (slot / kBlk) * rb * kBlk + (slot % kBlk);
        for (size_t gi = 0; gi < rb; ++gi) base[gi * kBlk] = src[gi];
        std::memcpy(&out.scales[slot], src + rb, 4);
        if (out.kind == 1) std::memcpy(&out.ids[slot], src + rb + 4, 8);
    };
    const size_t tail_row = rb + 4 + g.id_bytes(1);
    for (size_t k = 0; k < n % kBlk; ++k) place_row(n_full * kBlk + k, d + hd.tail_at + k * tail_row);
    for (const auto &op : hd.ops) place_row(op.first, d + op.second);   // pending redo writes (io_v7.rs:64-69)
    for (size_t i = 0; i < n; ++i)
        if (!std::isfinite(out.scales[i]) || !(out.scales[i] >= 0.f) || out.scales[i] > 1e22f) { error = "stored scale " + std::to_string(i) + " invalid"; return false; }
    return true;
}


// ---- incremental sync ----

namespace {
Geo geo_of(const V7SyncSource &src) { return Geo{src.kind, src.bits, src.dim, src.n_calib}; }

// codes | scale | id of one slot, as a tail row or a redo op carries them (io_v7.rs header_slot :560-583)
void put_row(std::vector<uint8_t> &out, const V7SyncSource &src, const Geo &g, size_t slot) {
    const uint8_t *codes;
    const float *scales;
    src.block(slot / kBlk, codes, scales);
    const size_t rb = g.row_bytes(), lane = slot % kBlk;
    for (size_t gi = 0; gi < rb; ++gi) out.push_back(codes[gi * kBlk + lane]);
    put<float>(out, scales[lane]);
    if (src.kind == 1) put<uint64_t>(out, src.ids[slot]);
}
}  // namespace

bool v7_plan_sync(const V7SyncSource &src, const V7Cursor &cursor, const std::unordered_set<size_t> &pending,
                  const std::unordered_set<size_t> &fresh, V7SyncPlan &plan) {
    const size_t old_blocks = size_t(cursor.n_synced) / kBlk, new_blocks = src.n / kBlk;
    const size_t live_rows = (old_blocks < new_blocks ? old_blocks : new_blocks) * kBlk;
    // Ops matter only for units committed under both states; a unit dirtied since the commit is never
    // touched on disk, all its ops (old and new) ride the new header instead.
    std::unordered_set<size_t> fresh_units;
    for (size_t s : fresh) if (s < live_rows) fresh_units.insert(s / kBlk);
    plan = V7SyncPlan();
    for (size_t s : pending)
        if (s < live_rows && !fresh_units.count(s / kBlk)) plan.materialise.push_back(s / kBlk);
    std::sort(plan.materialise.begin(), plan.materialise.end());
    plan.materialise.erase(std::unique(plan.materialise.begin(), plan.materialise.end()), plan.materialise.end());
    for (size_t s : pending) if (s < live_rows && fresh_units.count(s / kBlk)) plan.carried.push_back(s);
    for (size_t s : fresh) if (s < live_rows) plan.carried.push_back(s);
    std::sort(plan.carried.begin(), plan.carried.end());
    plan.carried.erase(std::unique(plan.carried.begin(), plan.carried.end()), plan.carried.end());
    if (plan.carried.size() > kMaxOps) return false;
    for (size_t s : plan.carried) {
        if (plan.groups.empty() || plan.groups.back().first != s / kBlk) plan.groups.push_back({s / kBlk, {}});
        plan.groups.back().second.push_back(s);
    }
    plan.append_from = old_blocks;
    plan.append_to = new_blocks;            // below append_from after a shrink: an empty range, written as it is
    plan.blocks_needed = plan.materialise;
    for (size_t b = plan.append_from; b < plan.append_to; ++b) plan.blocks_needed.push_back(b);
    for (const auto &grp : plan.groups) plan.blocks_needed.push_back(grp.first);
    if (src.n % kBlk) plan.blocks_needed.push_back(src.n / kBlk);
    std::sort(plan.blocks_needed.begin(), plan.blocks_needed.end());
    plan.blocks_needed.erase(std::unique(plan.blocks_needed.begin(), plan.blocks_needed.end()), plan.blocks_needed.end());
    return true;
}

void v7_build_sync(const V7SyncSource &src, const V7Cursor &cursor, const V7SyncPlan &plan, size_t clear_used,
                   std::vector<V7Batch> &batches) {
    const Geo g = geo_of(src);
    const uint64_t gen = cursor.gen + 1;
    const size_t rb = g.row_bytes();
    // One batch, one fsync: the header's delta descriptor names every unit written here and the digest of
    // their bytes, so a commit that reaches the disk before its data is detected at load.
    const size_t n_written = plan.materialise.size() + (plan.append_to > plan.append_from ? plan.append_to - plan.append_from : 0);
    PieceDigest digest(8 + n_written * (4 + g.unit_len()));
    digest.push(reinterpret_cast<const uint8_t *>(&gen), 8);
    V7Batch batch;
    auto write_unit = [&](size_t b) {
        const uint8_t *codes;
        const float *scales;
        src.block(b, codes, scales);
        V7Write w;
        w.offset = g.unit_at(b);
        w.bytes.reserve(g.unit_len());
        w.bytes.insert(w.bytes.end(), codes, codes + rb * kBlk);
        for (size_t l = 0; l < kBlk; ++l) put<float>(w.bytes, scales[l]);
        if (src.kind == 1)
            for (size_t l = 0; l < kBlk; ++l) put<uint64_t>(w.bytes, src.ids[b * kBlk + l]);
        const uint32_t b32 = uint32_t(b);
        digest.push(reinterpret_cast<const uint8_t *>(&b32), 4);
        digest.push(w.bytes.data(), w.bytes.size());
        batch.push_back(std::move(w));
    };
    for (size_t b : plan.materialise) write_unit(b);
    for (size_t b = plan.append_from; b < plan.append_to; ++b) write_unit(b);
    const uint32_t delta_crc = digest.finish();

    // The commit: generation g lives in slot g % 2, so this only ever overwrites the slot of generation g - 1.
    const size_t slot = size_t(gen % 2);
    V7Write hdr;
    hdr.offset = g.hdr_at(slot);
    std::vector<uint8_t> &h = hdr.bytes;
    put<uint64_t>(h, gen);
    put<uint64_t>(h, uint64_t(src.n));
    for (size_t r = src.n - src.n % kBlk; r < src.n; ++r) put_row(h, src, g, r);
    put<uint32_t>(h, uint32_t(plan.groups.size()));
    for (const auto &grp : plan.groups) {
        put<uint32_t>(h, uint32_t(grp.first));
        h.push_back(uint8_t(grp.second.size()));
        for (size_t s : grp.second) {
            h.push_back(uint8_t(s % kBlk));
            put_row(h, src, g, s);
        }
    }
    put<uint32_t>(h, uint32_t(plan.materialise.size()));
    for (size_t b : plan.materialise) put<uint32_t>(h, uint32_t(b));
    put<uint32_t>(h, uint32_t(plan.append_from));
    put<uint32_t>(h, uint32_t(plan.append_to));
    put<uint32_t>(h, delta_crc);
    put<uint32_t>(h, crc32c_split(h.data(), h.size()));
    batch.push_back(std::move(hdr));

    batches.clear();
    if (clear_used) {
        // A rejected header of this generation still sits in the slot: wipe all it occupies behind a barrier
        // of its own, and leave a generation whose parity disagrees with the slot so that the wiped slot is
        // refused outright (io_v7.rs:775-803).
        size_t len = clear_used < 8 ? 8 : clear_used;
        if (len > g.hdr_len()) len = g.hdr_len();
        V7Write wipe;
        wipe.offset = g.hdr_at(slot);
        wipe.bytes.assign(len, 0);
        const uint64_t wrong = (gen % 2) ^ 1;
        std::memcpy(wipe.bytes.data(), &wrong, 8);
        batches.push_back(V7Batch{std::move(wipe)});
    }
    batches.push_back(std::move(batch));
}

namespace {
bool pwrite_all(int fd, const uint8_t *d, size_t n, uint64_t off) {
    while (n) {
        const ssize_t w = ::pwrite(fd, d, n, off_t(off));
        if (w <= 0) return false;
        d += w; n -= size_t(w); off += uint64_t(w);
    }
    return true;
}
bool pread_all(int fd, uint8_t *d, size_t n, uint64_t off) {
    while (n) {
        const ssize_t r = ::pread(fd, d, n, off_t(off));
        if (r <= 0) return false;
        d += r; n -= size_t(r); off += uint64_t(r);
    }
    return true;
}
struct Fd {
    int fd;
    ~Fd() { if (fd >= 0) ::close(fd); }
};
}  // namespace

bool v7_run_sync(const char *path, const std::vector<V7Batch> &batches, std::string &error) {
    Fd f{::open(path, O_RDWR)};
    if (f.fd < 0) { error = std::string("cannot open ") + path; return false; }
    for (const V7Batch &batch : batches) {
        for (const V7Write &w : batch)
            if (!pwrite_all(f.fd, w.bytes.data(), w.bytes.size(), w.offset)) { error = std::string("write to ") + path + " failed"; return false; }
        if (::fsync(f.fd) != 0) { error = std::string("fsync of ") + path + " failed"; return false; }
    }
    return true;
}

V7CursorState v7_cursor_state(const char *path, const V7Cursor &cursor, const V7SyncSource &geometry, size_t &stale_used,
                              std::string &error) {
    stale_used = 0;
    const Geo g = geo_of(geometry);
    Fd f{::open(path, O_RDONLY)};
    if (f.fd < 0) {
        if (errno == ENOENT) return V7_CURSOR_REPLACED;
        error = std::string("cannot open ") + path;
        return V7_CURSOR_IO_ERROR;
    }
    struct stat st;
    if (::fstat(f.fd, &st) != 0) { error = std::string("cannot stat ") + path; return V7_CURSOR_IO_ERROR; }
    const size_t file_len = size_t(st.st_size);
    uint8_t head[19];
    if (file_len < sizeof head || !pread_all(f.fd, head, sizeof head, 0)) return V7_CURSOR_REPLACED;
    if (std::memcmp(head, kMagic, 4) != 0 || head[4] != kRevision) return V7_CURSOR_REPLACED;
    uint64_t file_nonce;
    std::memcpy(&file_nonce, head + 11, 8);
    if (file_nonce != cursor.nonce) return file_nonce == 0 ? V7_CURSOR_REPLACED : V7_CURSOR_FOREIGN;

    // Both header slots, newest first.
    std::vector<ParsedHeader> cands;
    std::vector<uint8_t> buf;
    for (size_t slot = 0; slot < 2; ++slot) {
        const size_t at = g.hdr_at(slot);
        if (at >= file_len) continue;
        // A commit that carries no redo ops uses only a short prefix of its slot: read that much first and the
        // whole slot only when the parse needs more (io_v7.rs hdr_probe_len :389-397).
        const size_t avail = file_len - at;
        const size_t full = g.hdr_len() < avail ? g.hdr_len() : avail;
        const size_t probe = 16 + 31 * (g.row_bytes() + 4 + g.id_bytes(1)) + 4 + 4 + kMaxOps * 4 + 12 + 4;
        for (size_t want = probe < full ? probe : full;; want = full) {
            buf.resize(want);
            if (!pread_all(f.fd, buf.data(), want, at)) break;
            ParsedHeader h;
            if (parse_header_bytes(buf.data(), want, at, g, slot, file_len, h)) { cands.push_back(std::move(h)); break; }
            if (want >= full) break;
        }
    }
    std::sort(cands.begin(), cands.end(), [](const ParsedHeader &a, const ParsedHeader &b) { return a.gen > b.gen; });
    if (!cands.empty() && cands.front().gen == cursor.gen) return V7_CURSOR_INTACT;
    // A header ahead of the cursor is either a sync of this index that did not finish (its delta fails and
    // the cursor's own commit is the adoptable one) or another writer's commit.
    for (const ParsedHeader &h : cands)
        if (h.gen > cursor.gen && h.used > stale_used) stale_used = h.used;
    std::vector<uint8_t> unit(g.unit_len());
    for (const ParsedHeader &h : cands) {
        const bool ok = delta_verified(h, g, [&](size_t u) -> const uint8_t * {
            if (g.unit_at(u) + g.unit_len() > file_len) return nullptr;
            return pread_all(f.fd, unit.data(), unit.size(), g.unit_at(u)) ? unit.data() : nullptr;
        });
        if (ok) {
            if (h.gen == cursor.gen) return V7_CURSOR_INTACT;
            stale_used = 0;
            return V7_CURSOR_FOREIGN;
        }
    }
    stale_used = 0;
    return V7_CURSOR_REPLACED;
}

uint64_t v7_fresh_nonce() {
    std::random_device rd;
    const uint64_t now = uint64_t(std::chrono::steady_clock::now().time_since_epoch().count());
    for (;;) {
        const uint64_t n = ((uint64_t(rd()) << 32) | rd()) ^ (now * 0x9E3779B97F4A7C15ull);
        if (n != 0) return n;                                  // zero marks a snapshot nobody syncs to
    }
}

bool v7_write_file_atomic(const char *path, const uint8_t *data, size_t len, std::string &error) {
    std::random_device rd;
    std::string tmp;
    int fd = -1;
    for (int attempt = 0; attempt < 8 && fd < 0; ++attempt) {
        char suffix[64];
        std::snprintf(suffix, sizeof suffix, ".tmp.%ld.%d.%08x", long(::getpid()), attempt, unsigned(rd()));
        tmp = std::string(path) + suffix;
        fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_EXCL, 0644);
        if (fd < 0 && errno != EEXIST) break;
    }
    if (fd < 0) { error = "cannot create a temporary file beside " + std::string(path); return false; }
    bool ok = pwrite_all(fd, data, len, 0) && ::fsync(fd) == 0;
    ok = (::close(fd) == 0) && ok;
    if (ok && std::rename(tmp.c_str(), path) != 0) ok = false;
    if (!ok) {
        std::remove(tmp.c_str());
        error = std::string("cannot write ") + path;
        return false;
    }
    // the rename itself is durable once the directory entry is (io.rs sync_parent_dir_after_commit)
    std::string dir(path);
    const size_t cut = dir.find_last_of('/');
    dir = cut == std::string::npos ? "." : (cut == 0 ? "/" : dir.substr(0, cut));
    const int dfd = ::open(dir.c_str(), O_RDONLY | O_DIRECTORY);
    if (dfd >= 0) { ::fsync(dfd); ::close(dfd); }
    return true;
}

}  // namespace tv
