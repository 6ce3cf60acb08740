// The reference's v7 container ("TV7\0", revision 2): full-image writer, loader and incremental sync, host only.
// Layout restated from turbovec/src/io_v7.rs: Geo :353-453, superblock :516-542, header_slot :549-599,
// unit_bytes :602-629, delta_digest :819-830, write_image :893-913, crc32 (CRC-32C, three-way split for
// inputs of 4096 bytes and more) :128-141.
#pragma once
#include <cstddef>
#include <cstdint>
#include <functional>
#include <string>
#include <unordered_set>
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
    uint64_t nonce = 0;                         // file identity; 0 = snapshot nobody syncs to (io_v7.rs UNCLAIMED_NONCE)
    uint64_t gen = 0;                           // read: generation of the adopted commit
    std::vector<size_t> pending_slots;          // read: slots whose redo ops ride the adopted header
};

uint32_t crc32c_split(const uint8_t *data, size_t len);      // the container's checksum
size_t v7_image_len(const V7Parts &p);
// Unclaimed snapshot (nonce 0, generation 0), identical to the reference's to_bytes()/write().
void v7_write_image(const V7Parts &p, std::vector<uint8_t> &out);
// Parses an image (either header slot, pending redo ops applied).  Returns false and sets `error`.
bool v7_read_image(const uint8_t *data, size_t len, V7Parts &out, std::string &error);


// ---- incremental sync (io_v7.rs plan_incremental :674-817, run_sync :865-876, cursor_state :1604-1700) ----

// The commit an index last wrote to, or loaded from, the file it is bound to (io_v7.rs SyncCursor).
struct V7Cursor {
    uint64_t gen = 0, n_synced = 0, calib_gen = 0, nonce = 0;
};

// Which units one incremental sync writes and which slots ride its header as redo ops.
struct V7SyncPlan {
    std::vector<size_t> materialise;                              // units whose pending ops are written into place
    size_t append_from = 0, append_to = 0;                        // units completed since the last commit
    std::vector<std::pair<size_t, std::vector<size_t>>> groups;   // (unit, slots): ops carried by the new header
    std::vector<size_t> carried;                                  // the same slots, flat and ascending
    std::vector<size_t> blocks_needed;                            // every block the serialisation reads
};

// Geometry and host-resident parts of the live index; codes and scales are fetched per 32-row block.
struct V7SyncSource {
    int kind = 0, bits = 4;
    size_t dim = 0, n = 0, n_calib = 0;
    const uint64_t *ids = nullptr;                                // slot -> id when kind == 1
    // sequential-blocked codes (32 * row bytes) and the 32 scales of `block`
    std::function<void(size_t block, const uint8_t *&codes, const float *&scales)> block;
};

struct V7Write {
    uint64_t offset;
    std::vector<uint8_t> bytes;
};
using V7Batch = std::vector<V7Write>;                             // all durable before the next batch starts

// False when the carried ops exceed the header's capacity: the caller rewrites the file whole.
bool v7_plan_sync(const V7SyncSource &src, const V7Cursor &cursor, const std::unordered_set<size_t> &pending,
                  const std::unordered_set<size_t> &fresh, V7SyncPlan &plan);
// The write batches of the planned sync.  `clear_used` > 0 asks for the repair barrier that destroys a
// rejected header of this generation (or a newer one) in the target slot before any data moves.
void v7_build_sync(const V7SyncSource &src, const V7Cursor &cursor, const V7SyncPlan &plan, size_t clear_used,
                   std::vector<V7Batch> &batches);
// Positioned writes, one fsync per batch.
bool v7_run_sync(const char *path, const std::vector<V7Batch> &batches, std::string &error);

enum V7CursorState { V7_CURSOR_INTACT = 0, V7_CURSOR_FOREIGN = 1, V7_CURSOR_REPLACED = 2, V7_CURSOR_IO_ERROR = 3 };
// Whether the file at `path` is still the one `cursor` describes.  For an intact file `stale_used` is the
// used length of a parseable header ahead of the cursor (0 when there is none).
V7CursorState v7_cursor_state(const char *path, const V7Cursor &cursor, const V7SyncSource &geometry, size_t &stale_used,
                              std::string &error);
// A fresh non-zero file identity (io.rs file_nonce).
uint64_t v7_fresh_nonce();
// Temp file beside `path`, fsync, rename over it, fsync of the directory (io.rs:14-27).
bool v7_write_file_atomic(const char *path, const uint8_t *data, size_t len, std::string &error);

}  // namespace tv
