#include "io_v7.hpp"

#include <cmath>
#include <cstring>

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
    put<uint64_t>(out, 0);                                   // unclaimed snapshot
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
    size_t n = 0, tail_at = 0;
    std::vector<std::pair<size_t, size_t>> ops;              // (slot, offset of codes in the file)
    std::vector<size_t> delta_units;
    uint32_t delta_crc = 0;
};

bool parse_header(const uint8_t *d, size_t len, const Geo &g, size_t slot, ParsedHeader &h) {
    const size_t at = g.hdr_at(slot);
    if (at + g.hdr_len() > len) return false;
    const uint8_t *b = d + at;
    const size_t cap = g.hdr_len();
    uint64_t gen, n64;
    if (!get(b, cap, 0, gen) || !get(b, cap, 8, n64)) return false;
    if (gen % 2 != slot) return false;
    const size_t n = size_t(n64);
    if (g.unit_at(n / kBlk) > len) return false;
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
    for (uint32_t u = from; u < to; ++u) h.delta_units.push_back(u);
    h.gen = gen; h.n = n; h.tail_at = at + 16;
    // delta check: the units this commit wrote are on disk as it wrote them (io_v7.rs:843-858)
    PieceDigest dg(8 + h.delta_units.size() * (4 + g.unit_len()));
    dg.push(reinterpret_cast<const uint8_t *>(&gen), 8);
    for (size_t u : h.delta_units) {
        if (g.unit_at(u + 1) > len) return false;
        const uint32_t u32 = uint32_t(u);
        dg.push(reinterpret_cast<const uint8_t *>(&u32), 4);
        dg.push(d + g.unit_at(u), g.unit_len());
    }
    return dg.finish() == h.delta_crc;
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

}  // namespace tv
