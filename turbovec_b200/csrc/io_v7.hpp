// The reference's v7 container ("TV7\0", revision 2): full-image writer and loader, host only.
// Layout restated from turbovec/src/io_v7.rs: Geo :353-453, superblock :516-542, header_slot :549-599,
// unit_bytes :602-629, delta_digest :819-830, write_image :893-913, crc32 (CRC-32C, three-way split for
// inputs of 4096 bytes and more) :128-141.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace tv {

struct V7Parts {
    int kind = 0;                 // 0 = positional index, 1 = id-mapped index
    int bits = 4;
    size_t dim = 0;
    size_t n = 0;
    std::vector<float> boundaries, centroids;   // 2^bits - 1, 2^bits
    std::vector<float> shift, scale;            // empty or dim each
    std::vector<uint8_t> blocked;               // ceil(n/32) * ngroups * 32, sequential-blocked
    std::vector<float> scales;                  // n
    std::vector<uint64_t> ids;                  // n when kind == 1
};

uint32_t crc32c_split(const uint8_t *data, size_t len);      // the container's checksum
size_t v7_image_len(const V7Parts &p);
// Unclaimed snapshot (nonce 0, generation 0), identical to the reference's to_bytes()/write().
void v7_write_image(const V7Parts &p, std::vector<uint8_t> &out);
// Parses an image (either header slot, pending redo ops applied).  Returns false and sets `error`.
bool v7_read_image(const uint8_t *data, size_t len, V7Parts &out, std::string &error);

}  // namespace tv
