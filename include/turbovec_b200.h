/*
 * turbovec_b200 — C ABI of the B200 (sm_100a) encode-and-scan library.
 *
 * The reference (a Rust crate) has no FFI seam for this path: its Python
 * binding calls the index types in process.  This header therefore mirrors
 * the reference's index-level API one to one, so that a Rust `extern "C"`
 * shim (or the pyo3 classes) can forward to it without reshaping arguments.
 * Every entry point names the reference function it replaces; paths are
 * relative to the reference project root.
 *
 * Conventions
 *  - All pointers are HOST pointers unless the name says `_device`.
 *  - Arrays are row-major and contiguous; the caller owns every buffer.
 *  - Every call returns a tv_status; 0 is success.  A failing call leaves the
 *    index exactly as it was (the reference's all-or-nothing contract,
 *    turbovec/src/lib.rs:889-930).  tv_last_error() gives the message.
 *  - Calls are synchronous: results are complete when the call returns.
 *  - A handle may be used from several threads, like the reference's index
 *    (`search(&self)`, mutation through `&mut self`; turbovec/src/lib.rs:22-52):
 *    searches hold the handle shared and overlap on the device (two at a
 *    time, each on its own stream and scratch; further ones wait), every
 *    call that changes the index is exclusive.
 *  - There is no CPU fallback: every compute entry point needs a CUDA device.
 */
#ifndef TURBOVEC_B200_H
#define TURBOVEC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tv_index tv_index;

/* Status codes.  One per error variant of turbovec/src/error.rs. */
typedef enum tv_status {
    TV_OK = 0,
    /* ConstructError, error.rs:166-183 (raised lib.rs:629-638) */
    TV_ERR_BIT_WIDTH_OUT_OF_RANGE = 1,
    TV_ERR_DIM_NOT_POSITIVE_MULTIPLE_OF_8 = 2,
    TV_ERR_DIM_TOO_LARGE = 3,
    /* AddError, error.rs:45-116 (raised lib.rs:1114-1148, id_map.rs:379-434) */
    TV_ERR_DIM_MISMATCH = 10,
    TV_ERR_ZERO_DIM = 11,
    TV_ERR_DIM_NOT_MULTIPLE_OF_8 = 12,
    TV_ERR_BUFFER_NOT_MULTIPLE_OF_DIM = 13,
    TV_ERR_IDS_COUNT_MISMATCH = 14,
    TV_ERR_ID_ALREADY_PRESENT = 15,
    TV_ERR_DUPLICATE_ID_IN_BATCH = 16,
    TV_ERR_INVALID_INPUT_VALUE = 17,
    /* SearchError, error.rs:234-275 (raised lib.rs:1363-1433, id_map.rs:672-677) */
    TV_ERR_ALLOWLIST_EMPTY = 20,
    TV_ERR_UNKNOWN_ID = 21,
    TV_ERR_QUERY_BUFFER_NOT_MULTIPLE_OF_DIM = 22,
    TV_ERR_INVALID_QUERY_VALUE = 23,
    TV_ERR_MASK_LENGTH_MISMATCH = 24,
    /* contract violations the reference panics on (lib.rs:718-721, 2869-2873) */
    TV_ERR_DIM_NOT_SET = 30,
    TV_ERR_SLOT_OUT_OF_RANGE = 31,
    TV_ERR_WRONG_INDEX_KIND = 32,
    /* FromPartsError, error.rs:324-433 (checks lib.rs:2383-2492) */
    TV_ERR_PARTS_INVALID = 40,
    /* CalibrateError, error.rs:516-588 */
    TV_ERR_CALIBRATE_SAMPLE_TOO_SMALL = 50,
    TV_ERR_CALIBRATE_DEGENERATE_SAMPLE = 51,
    TV_ERR_CALIBRATE_NOT_EMPTY = 52,    /* no longer returned: a populated index is refitted */
    /* this library */
    TV_ERR_INVALID_ARGUMENT = 90,
    TV_ERR_CUDA = 91,
    TV_ERR_OUT_OF_MEMORY = 92,
    TV_ERR_UNSUPPORTED = 93,
    TV_ERR_DEVICE_TIMEOUT = 94,
    TV_ERR_IO = 95,                     /* a file could not be opened, read, written or made durable */
    TV_ERR_SYNC_FOREIGN_FILE = 96       /* tv_sync: another writer advanced or replaced the bound file */
} tv_status;

/* Index kinds: turbovec/src/lib.rs:295 (TurboQuantIndex), id_map.rs:221 (IdMapIndex). */
enum { TV_KIND_POSITIONAL = 0, TV_KIND_IDMAP = 1 };

/*
 * Score arithmetic.  The reference picks one of its kernel families from the
 * host CPU's features (turbovec/src/pack.rs:1189-1263, search.rs:2975-2980);
 * each rounds scores differently.  AUTO is what an x86 host with AVX-512
 * VBMI+VNNI runs: permute-dot int8 for 4-bit when ngroups % 4 == 0, the u8
 * LUT scan with (f32)isum*scale+bias for 2/3-bit when ngroups % 4 == 0, and
 * the u8 LUT scan with one fma per 256 byte-groups otherwise.
 */
enum {
    TV_SCORE_AUTO = 0,
    TV_SCORE_PERMUTE_DOT = 1,
    TV_SCORE_LUT_MULADD = 2,
    TV_SCORE_LUT_FLUSH = 3
};

/* Options for tv_set_option. */
enum {
    TV_OPT_SCORE_MODE = 1,      /* one of TV_SCORE_* */
    TV_OPT_MMA_MIN_BATCH = 2,   /* query batches of at least this size use the tensor-memory scan; 0 = never;
                                 * -1 (default) = measured switch points: permute-dot 17 with the int8 copy of the index
                                 * (TV_OPT_TC_EXPANDED) and 33 without it, u8-LUT families 8 */
    TV_OPT_FORCE_CAREFUL = 3,   /* 1: run the candidate-overflow recovery schedule always (testing) */
    TV_OPT_TC_TILES = 4,        /* accumulator tiles of 128 vectors per query slab in the tensor-memory scan: 1 or 2 */
    TV_OPT_INGEST_PIPELINE = 5, /* 1 (default): whole code blocks are encoded by the pipelined ingest kernel; 0: never;
                                 * 2: pipelined, and every reconstruction sum walks the sequential chains (testing) */
    TV_OPT_PD_SPLIT = 6,        /* 1 (default): batches of up to 32 queries on 4-bit permute-dot indexes look the int8
                                 * levels up with one byte-permute per four codes and half-table (two exact integer
                                 * contractions, subtracted); 0: merged lookup, one contraction (testing) */
    TV_OPT_SMALL_SCAN = 7,      /* permute-dot batches of up to 16 queries: -1 = the general small-batch kernel; otherwise
                                 * a variant of the stream-shaped kernel (bits 0-1: ring depth 3 / 4 / 6 stages per warp,
                                 * bit 2: swizzled tensor copies instead of plain bulk copies; default 5).  Results are identical. */
    TV_OPT_FAIL_NEXT = 8,       /* testing: the n-th guarded device allocation / upload from now on reports an
                                 * out-of-memory failure instead of running (1 = the next one); 0 disarms */
    TV_OPT_TC_WIDE = 10,        /* 1 (default): batches of more than 256 queries run the tensor-memory scan whose work items
                                 * take two query groups per expanded code slab; 0: one group per item.  Identical results. */
    TV_OPT_TC_EXPANDED = 11,    /* permute-dot batches on the tensor-memory scan read an int8 copy of the index (one level per
                                 * coordinate: twice the bytes of the 4-bit codes) instead of expanding codes in the kernel.
                                 * 1 (default): when the copy fits with a tenth of the device left free; 0: never (drops the
                                 * copy); 2: always, a search fails when it does not fit.  The copy is built and kept current
                                 * lazily by the searches that use it.  Identical results. */
    TV_OPT_EXPANDED_BYTES = 12, /* read-only: bytes the int8 copy holds right now (0 = none) */
    TV_OPT_DENSE_PAIR = 13      /* 1 (default): the scan over the int8 copy runs on CTA pairs (tcgen05 cta_group::2: half the
                                 * query bytes per SM); 0: one CTA per work item.  Identical results. */
};

/* ---- construction: TurboQuantIndex::new / new_lazy (lib.rs:629, 670), IdMapIndex::new (id_map.rs:278) ---- */
/* dim == 0 creates a lazy index whose dimension is fixed by the first add.  device = CUDA ordinal. */
int tv_index_create(size_t dim, int bit_width, int kind, int device, tv_index **out);
void tv_index_destroy(tv_index *h);

/* Message of the most recent failing call on this handle (or of the last failed create when h == NULL). */
const char *tv_last_error(const tv_index *h);
/* Offender of the last TV_ERR_INVALID_INPUT_VALUE / TV_ERR_INVALID_QUERY_VALUE (error.rs:104-116, 262-270),
 * or id of the last TV_ERR_ID_ALREADY_PRESENT / DUPLICATE_ID_IN_BATCH / UNKNOWN_ID in *id. */
void tv_error_detail(const tv_index *h, size_t *vector_index, size_t *coord_index, float *value, uint64_t *id);

/* ---- introspection: len / dim_opt / bit_width (lib.rs:3031-3064) ---- */
size_t tv_len(const tv_index *h);
size_t tv_dim(const tv_index *h);      /* 0 while lazy */
int tv_bit_width(const tv_index *h);
int tv_kind(const tv_index *h);
int tv_set_option(tv_index *h, int option, int64_t value);
int64_t tv_get_option(const tv_index *h, int option);

/* ---- ingest: add_2d (lib.rs:1114-1210) -> encode_and_append (lib.rs:823) -> encode::encode (encode.rs:510) ---- */
int tv_add(tv_index *h, const float *vectors, size_t n, size_t dim);
/* add_with_ids_2d (id_map.rs:373-469); TV_KIND_IDMAP only. */
int tv_add_with_ids(tv_index *h, const float *vectors, size_t n, size_t dim, const uint64_t *ids);
/* Same as tv_add but `vectors` is device memory on the handle's device.  The finite/|x|<1e16 check of
 * encode.rs:58-74 runs on the device.  Used when the producer already lives on the GPU. */
int tv_add_device(tv_index *h, const float *vectors_device, size_t n, size_t dim);
/* tv_add_with_ids with the rows in device memory; `ids` stays a host array (ids never reach the device). */
int tv_add_with_ids_device(tv_index *h, const float *vectors_device, size_t n, size_t dim, const uint64_t *ids);

/* ---- removal: swap_remove (lib.rs:2864-3028), IdMapIndex::remove (id_map.rs:520-567) ----
 * Both return once the move of the last row into the freed slot is enqueued on the handle's stream; every
 * later call on the handle is ordered after it. */
int tv_swap_remove(tv_index *h, size_t slot, size_t *moved_from);
int tv_remove(tv_index *h, uint64_t id, int *removed);
/* One stored row as its byte-groups in group order plus its scale: pack::read_code / write_code over a lane
 * (pack.rs:1113-1160).  Used to move a row between device shards when swap_remove crosses GPUs. */
int tv_get_row(const tv_index *h, size_t slot, uint8_t *groups_out, size_t capacity, float *scale_out);
int tv_set_row(tv_index *h, size_t slot, const uint8_t *groups, size_t count, float scale);
int tv_contains(const tv_index *h, uint64_t id, int *present);         /* id_map.rs:593 */
/* Copies slot_to_id[0..len) (id_map.rs:631 iter_ids order). */
int tv_ids(const tv_index *h, uint64_t *ids_out, size_t capacity);

/* ---- search: try_search_with_mask (lib.rs:1345-1485) -> search::search (search.rs:3206) ----
 * mask_bool: NULL or `mask_len` bytes, non-zero = slot allowed (must equal len, lib.rs:1427-1433).
 * scores_out / slots_out: nq * min(k, len) entries; row stride is *k_eff = min(k, len, n_allowed).
 * A lazy or empty index yields k_eff = 0 and TV_OK (lib.rs:1355-1402). */
int tv_search(tv_index *h, const float *queries, size_t nq, size_t dim, size_t k, const uint8_t *mask_bool,
              size_t mask_len, float *scores_out, int64_t *slots_out, size_t *k_eff);
/* Same with the mask already packed: bit i of little-endian u64 word i/64 = slot i (search.rs:2996-3004). */
int tv_search_mask_words(tv_index *h, const float *queries, size_t nq, size_t dim, size_t k,
                         const uint64_t *mask_words, size_t n_words, float *scores_out, int64_t *slots_out,
                         size_t *k_eff);
/* try_search_with_allowlist (id_map.rs:664-712); allow_ids == NULL means unfiltered.  ids_out receives ids. */
int tv_search_allowlist(tv_index *h, const float *queries, size_t nq, size_t dim, size_t k,
                        const uint64_t *allow_ids, size_t n_allow, float *scores_out, uint64_t *ids_out,
                        size_t *k_eff);
/* Device-resident variant: queries, optional mask words, scores and slots all in device memory.
 * Nothing crosses PCIe except the launch parameters and one status word. */
int tv_search_device(tv_index *h, const float *queries_device, size_t nq, size_t k,
                     const uint64_t *mask_words_device, float *scores_out_device, int64_t *slots_out_device,
                     size_t *k_eff);

/* ---- one filter, many searches.  The reference rebuilds the slot mask from the allowlist on every call
 * (id_map.rs:670-683, lib.rs:1435-1456: |allowlist| hash lookups plus a pass over all slots); these entry
 * points do that work once and keep the packed mask, the list of code blocks that hold an allowed slot and
 * the allowed count on the device.  Any call that changes the index drops the prepared mask; searching with
 * a dropped or missing one fails with TV_ERR_INVALID_ARGUMENT.  No reference counterpart.
 * tv_mask_prepare_device: packed words in device memory (bit i of word i/64 = slot i, ceil(len/64) words).
 * tv_mask_prepare_words: the same words in host memory.  tv_mask_prepare_allowlist: ids (TV_KIND_IDMAP), with
 * the allowlist errors of tv_search_allowlist.  tv_search_prepared / tv_search_device_prepared: as tv_search /
 * tv_search_device under the prepared mask; ids_out (may be NULL) needs an id-mapped index. ---- */
int tv_mask_prepare_device(tv_index *h, const uint64_t *mask_words_device);
int tv_mask_prepare_words(tv_index *h, const uint64_t *mask_words, size_t n_words);
int tv_mask_prepare_allowlist(tv_index *h, const uint64_t *allow_ids, size_t n_allow);
int tv_search_prepared(tv_index *h, const float *queries, size_t nq, size_t dim, size_t k, float *scores_out,
                       int64_t *slots_out, uint64_t *ids_out, size_t *k_eff);
int tv_search_device_prepared(tv_index *h, const float *queries_device, size_t nq, size_t k,
                              float *scores_out_device, int64_t *slots_out_device, size_t *k_eff);

/* ---- slot-sharded search over several GPUs (one process per GPU).  No reference counterpart: the reference
 * is a single-host library; these two calls are the per-rank half and the merge half of a sharded search. ----
 * tv_search_device_keys: like tv_search_device, but each result is one 64-bit key = (order-preserving image of
 * the score, descending) << 32 | (slot + slot_offset); ascending key order is the reference's result order
 * (score descending, slot ascending, search.rs:236-252).  Rows are k keys wide, padded with TV_EMPTY_KEY.
 * slot_offset = the shard's first global slot; slot_offset + len must not exceed 2^32.
 * tv_merge_keys_device: keys[n_lists][nq][k] (e.g. the all-gathered rows of every rank) -> per query the k
 * best, decoded to scores and global slots (rows of k; unused places hold (-inf, 0)); runs on `stream`
 * (a cudaStream_t, may be null) of `device` without synchronising; n_lists * k <= 8192. */
#define TV_EMPTY_KEY 0xffffffffffffffffull
int tv_search_device_keys(tv_index *h, const float *queries_device, size_t nq, size_t k,
                          const uint64_t *mask_words_device, uint64_t slot_offset, uint64_t *keys_out_device,
                          size_t *k_eff);
int tv_merge_keys_device(int device, const uint64_t *keys_device, size_t n_lists, size_t nq, size_t k,
                         float *scores_out_device, int64_t *slots_out_device, void *stream);
/* The same merge for shards that own chunks of `chunk_slots` global slots round-robin (list r owns the chunks
 * r, r + n_lists, ...: appends stay balanced at any length): the lists carry LOCAL slots (slot_offset 0), which
 * become global slots = ((local / chunk_slots) * n_lists + r) * chunk_slots + local % chunk_slots before the
 * merge, so that ties break by the global slot as in the reference.  chunk_slots a multiple of 32. */
int tv_merge_keys_device_chunked(int device, const uint64_t *keys_device, size_t n_lists, size_t nq, size_t k,
                                 size_t chunk_slots, float *scores_out_device, int64_t *slots_out_device, void *stream);

/* ---- id tables without vectors: the slot_to_id / id_to_slot pair IdMapIndex keeps around its inner index
 * (id_map.rs:221-272).  A slot-sharded id-mapped index numbers slots globally, so every rank keeps a replica of
 * these tables and applies the same calls in the same order; they never touch a device.
 * add: id checks of add_with_ids_2d in the reference's order, nothing changes on error (id_map.rs:396-434).
 * remove: id_map.rs:520-567; *slot = the freed slot, *moved_from = the slot whose row takes its place.
 * resolve: allowlist ids -> global slots with the allowlist errors of id_map.rs:670-683 (TV_ERR_ALLOWLIST_EMPTY,
 * TV_ERR_UNKNOWN_ID for the first unknown id in list order).  ids_of: slots -> ids (id_map.rs:695-705). ---- */
typedef struct tv_idtable tv_idtable;
int tv_idtable_create(tv_idtable **out);
void tv_idtable_destroy(tv_idtable *t);
size_t tv_idtable_len(const tv_idtable *t);
const char *tv_idtable_last_error(const tv_idtable *t, uint64_t *id);
int tv_idtable_add(tv_idtable *t, const uint64_t *ids, size_t n);
int tv_idtable_truncate(tv_idtable *t, size_t n);
int tv_idtable_remove(tv_idtable *t, uint64_t id, int *removed, uint64_t *slot, uint64_t *moved_from);
int tv_idtable_contains(const tv_idtable *t, uint64_t id, int *present);
int tv_idtable_resolve(const tv_idtable *t, const uint64_t *ids, size_t n, uint64_t *slots_out);
int tv_idtable_ids_of(const tv_idtable *t, const int64_t *slots, size_t n, uint64_t *ids_out);
int tv_idtable_ids(const tv_idtable *t, uint64_t *ids_out, size_t capacity);

/* ---- one handle over several GPUs of one process (csrc/multi.cpp).  No reference counterpart: the reference is a
 * single-host library.  The handle owns one positional index per listed device (the same device may be listed more
 * than once) and deals global slots to them round-robin in chunks of 32 * chunk_blocks slots (0 = 1,024 blocks; must
 * be even), so every call below has the meaning of its single-device namesake over GLOBAL slot numbers: add /
 * add_with_ids (lib.rs:1114, id_map.rs:373; all or nothing), swap_remove / remove (lib.rs:2864, id_map.rs:520; the
 * globally last row moves into the hole, across devices if need be), search with a bool mask over global slots
 * (lib.rs:1345) or an allowlist of ids (id_map.rs:664), contains / ids (id_map.rs:593, 631).  A search runs every
 * shard's scan at the same time (tv_search_device_keys, one host thread per shard) and merges the result keys on the
 * first device (tv_merge_keys_device_chunked); results are identical to one index holding all the rows.
 * kind = TV_KIND_IDMAP keeps the id tables (tv_idtable_*) beside the shards.  Limits: shards * min(k, len) <= 8192;
 * one call at a time per handle (the handle serialises them).  tv_multi_shard gives a shard's index for options and
 * inspection (do not add to or remove from it directly). ---- */
typedef struct tv_multi tv_multi;
int tv_multi_create(size_t dim, int bit_width, int kind, const int *device_ids, int n_devices, size_t chunk_blocks, tv_multi **out);
void tv_multi_destroy(tv_multi *m);
const char *tv_multi_last_error(const tv_multi *m);        /* m == NULL: the last failed create of this thread */
uint64_t tv_multi_error_id(const tv_multi *m);             /* id of the last id error (already present / duplicate / unknown) */
size_t tv_multi_len(const tv_multi *m);
int tv_multi_shards(const tv_multi *m);
tv_index *tv_multi_shard(tv_multi *m, int i);
int tv_multi_add(tv_multi *m, const float *vectors, size_t n, size_t dim);
int tv_multi_add_with_ids(tv_multi *m, const float *vectors, size_t n, size_t dim, const uint64_t *ids);
int tv_multi_swap_remove(tv_multi *m, size_t slot, size_t *moved_from);
int tv_multi_remove(tv_multi *m, uint64_t id, int *removed);
int tv_multi_contains(const tv_multi *m, uint64_t id, int *present);
int tv_multi_ids(const tv_multi *m, uint64_t *ids_out, size_t capacity);
int tv_multi_search(tv_multi *m, const float *queries, size_t nq, size_t dim, size_t k, const uint8_t *mask_bool, size_t mask_len,
                    float *scores_out, int64_t *slots_out, size_t *k_eff);
int tv_multi_search_allowlist(tv_multi *m, const float *queries, size_t nq, size_t dim, size_t k, const uint64_t *allow_ids,
                              size_t n_allow, float *scores_out, uint64_t *ids_out, size_t *k_eff);

/* Search that performs no allocation of any kind.  This entry point has no counterpart in the reference:
 * it exists for callers that must not reach the CUDA allocator while they serve — latency-critical loops
 * (cudaMalloc locks the device and may synchronise it), processes whose device memory is fully handed out,
 * frameworks that forbid allocator traffic after warm-up.  Same contract as tv_search_device (unfiltered;
 * queries, scores and slots in device memory; output row stride *k_eff), but all scratch sits in one fixed
 * 1.25 MiB array inside the library image, resident on every GPU that loads the library until exit.
 * Limits: nq <= 8, k <= 128, index dim <= 4096 (and, for 2/3-bit and other u8-LUT geometries, tables of one
 * query that fit in shared memory: 32 * ngroups bytes <= 226 KB); larger requests fail with TV_ERR_UNSUPPORTED
 * and a message.  It runs the chunk schedule of tv_search_device on the CUDA-core scan kernels (a handful of
 * launches whatever the index size; a 10 M x 1536 4-bit index answers in about the time of tv_search_device
 * at the same batch), and an adversarial vector order that overflows a candidate list is redone in bounded
 * chunks, still without memory beyond the array.  The index tables must exist (tv_prepare or a previous add).
 * The first call on each device resolves the array's device address, and the first call with a given batch
 * size and score mode loads that kernel: warm up with the batch sizes you serve, before any stream capture
 * begins.  All calls share the array, which keeps whatever the previous call left; within a process calls are
 * serialised, and work from other sources that touches the same array while a call is in flight would race
 * with it. */
int tv_search_device_noalloc(tv_index *h, const float *queries_device, size_t nq, size_t k,
                             float *scores_out_device, int64_t *slots_out_device, size_t *k_eff);

/* ---- warm-up: prepare (lib.rs:1496) — builds tables and caches the first search would build ---- */
int tv_prepare(tv_index *h);

/* ---- raw parts: codes_blocked_seq / scales / packed_codes / from_parts (lib.rs:2088, 2533, 2528, 2371) ----
 * blocked: ceil(len/32) * ngroups * 32 bytes in the reference's sequential-blocked layout
 * (pack.rs:340-361); scales: len floats. */
size_t tv_blocked_bytes(const tv_index *h);
int tv_export_blocked(const tv_index *h, uint8_t *blocked_out, size_t blocked_capacity, float *scales_out,
                      size_t scales_capacity);
/* Bit-plane rows as packed_codes() returns them: len * bit_width*dim/8 bytes (encode.rs:1464-1470). */
int tv_export_packed(const tv_index *h, uint8_t *packed_out, size_t capacity);
/* from_parts: replaces the contents of an EMPTY index with n rows given as bit-plane rows + scales
 * (+ ids for TV_KIND_IDMAP, else NULL).  Validation follows lib.rs:2383-2492. */
int tv_import_packed(tv_index *h, size_t dim, const uint8_t *packed, size_t n, const float *scales,
                     const uint64_t *ids);
/* Codebook the index encodes against: codebook_for_write (lib.rs:2108).  boundaries: 2^bits-1, centroids: 2^bits. */
int tv_codebook(tv_index *h, float *boundaries_out, float *centroids_out);
/* Rotate rows exactly as queries are rotated (Rotation::apply, rotation.rs:202) — diagnostic entry point. */
int tv_rotate(tv_index *h, const float *rows, size_t n, size_t dim, float *rotated_out);

/* ---- persistence: to_bytes / from_bytes / write / load (lib.rs:2167, 2207, 2055, 2235) ----
 * The image is the reference's v7 container (turbovec/src/io_v7.rs), byte for byte the snapshot the
 * reference's to_bytes()/write() produce for the same index state, so files interchange.  Files that
 * incremental syncs have advanced load with their pending redo ops applied. */
/* The container's checksum: CRC-32C, and for inputs of 4096 bytes or more the CRC-32C of the three CRCs of the
 * input's thirds (io_v7.rs:128-141). */
uint32_t tv_crc32c(const uint8_t *data, size_t len);
size_t tv_image_bytes(const tv_index *h);
int tv_to_bytes(const tv_index *h, uint8_t *out, size_t capacity);
int tv_from_bytes(const uint8_t *data, size_t len, int expect_kind, int device, tv_index **out);
int tv_write(const tv_index *h, const char *path);
int tv_load(const char *path, int expect_kind, int device, tv_index **out);
/* Incremental persistence (lib.rs:1737 `sync`, id_map.rs:867; io_v7.rs plan_incremental :674, run_sync :865,
 * cursor_state :1604).  The first sync of a path - or a sync to another path than the last one, after a
 * calibration, over a file that was replaced, or with more than 1,024 dirtied committed slots - writes the whole
 * index as a fresh container under a new random file identity (temporary file, fsync, rename).  Every other
 * sync is one batch of positioned writes and one fsync: the 32-row units completed since the last commit,
 * the units whose pending redo ops can now be written into place, and the alternate commit header with the
 * tail rows, the redo ops of units dirtied since the last commit and the digest of the units just written.
 * An index loaded by tv_load from a file that a sync has claimed is bound to it; a snapshot written by
 * tv_write is not.  Returns TV_ERR_SYNC_FOREIGN_FILE when the bound file carries another identity or a commit
 * this index did not write, TV_ERR_IO when the file cannot be written (the binding is dropped: the next sync
 * rewrites the file whole), TV_ERR_DIM_NOT_SET for a lazy index. */
int tv_sync(tv_index *h, const char *path);
/* The binding tv_sync keeps (tests): whether the index is bound to a file, the generation of its last commit,
 * how many slots ride that commit's header as redo ops, how many committed slots were dirtied since. */
int tv_sync_state(const tv_index *h, int *bound, uint64_t *generation, size_t *n_pending, size_t *n_fresh);
/* The planner of an incremental sync on plain arrays, host only (tests; io_v7.rs plan_incremental :674-735):
 * from the rows of the last commit, the live row count, the slots whose redo ops ride the committed header and
 * the committed slots dirtied since, the units to write into place and the slots the new header carries (both
 * ascending; the arrays' capacities come in through *n_materialise / *n_carried) and the appended unit range.
 * TV_ERR_UNSUPPORTED when more than 1,024 slots would be carried (the caller rewrites the file whole). */
int tv_v7_plan_sync(size_t n_synced, size_t n, const size_t *pending, size_t n_pending, const size_t *fresh,
                    size_t n_fresh, size_t *materialise_out, size_t *n_materialise, size_t *carried_out,
                    size_t *n_carried, size_t *append_from, size_t *append_to);

/* ---- TQ+ calibration: calibrate_2d (lib.rs:2599-2723); on a populated index every stored row is re-encoded from
 * its own codes under the new pair (reencode_stored_rows, lib.rs:2760-2832); tqplus_shift/scale (lib.rs:2535-2545) ---- */
int tv_calibrate(tv_index *h, const float *sample, size_t n, size_t dim);
int tv_calibration(const tv_index *h, float *shift_out, float *scale_out, size_t capacity, int *is_calibrated);
int tv_set_calibration(tv_index *h, size_t dim, const float *shift, const float *scale);

/* ---- instrumentation ---- */
/* Kernels of this library launched on this handle since creation (for benchmark bookkeeping). */
uint64_t tv_launch_count(const tv_index *h);
/* Device time of the kernels of the last search / add call, from CUDA events on the handle's stream (ms). */
float tv_last_kernel_ms(const tv_index *h);
/* Summed device time (ms) of the dominant kernel's launches in the last call — the block scan for a search,
 * the ingest kernel for an add — each launch bracketed by its own pair of events; *launches = how many. */
float tv_last_main_kernel_ms(const tv_index *h, int *launches);
const char *tv_version(void);
/* Measures the device's int8 tensor rate for this library's MMA form (tcgen05 kind::i8, M = 128, N = 256, K = 32,
 * operands in shared memory, accumulators in tensor memory; no loads, no epilogue): ops per second with a
 * multiply-add counted as 2.  About 25 ms.  The roofline the large-batch permute-dot scan is reported against;
 * no reference counterpart. */
int tv_measure_int8_peak(int device, double *ops_per_second);
/* The same kernel launched back to back for `seconds` (at most 10): the rate over the second half of that time, i.e. what
 * the device sustains once its power limit acts.  seconds <= 0: the burst figure of tv_measure_int8_peak. */
int tv_measure_int8_peak_for(int device, double seconds, double *ops_per_second);
/* Host-side evaluation of the quantisation grid that the pipelined ingest kernel builds from a codebook's
 * boundaries (`count` ascending values, at most 15): codes_out[i] = number of boundaries strictly below
 * values[i] (encode.rs:1447-1451), looked up exactly as the kernel does.  Returns TV_ERR_UNSUPPORTED when the
 * boundaries admit no grid (the kernel is then not used).  No reference counterpart: it exists so that the
 * table construction can be checked against a plain count without a device. */
int tv_quantise_grid_lookup(const float *boundaries, int count, const float *values, size_t n, uint8_t *codes_out);
/* Host-side check of the shared-memory layout through which the two rotation rounds of the pipelined ingest
 * kernel exchange a row (built per dimension by edge-colouring the store/gather instruction graph): the
 * largest number of lanes of one warp instruction that fall on one bank, for the stores and for the round-2
 * gathers, with plain rows and with the layout (1 = conflict-free).  No reference counterpart; for tests. */
int tv_exchange_layout_conflicts(size_t dim, int *store_plain, int *gather_plain, int *store_layout, int *gather_layout);

#ifdef __cplusplus
}
#endif
#endif /* TURBOVEC_B200_H */
