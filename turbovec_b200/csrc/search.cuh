// Launch interface of the search-side kernels (see search.cu).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace tv {

// Float epilogues of the reference's kernel families (turbovec/src/search.rs:1523, 1176, 1596).
enum ScoreMode : int { kModePermuteDot = 1, kModeLutMulAdd = 2, kModeLutFlush = 3 };

struct QueryPrepParams {
    const float *queries;          // [nq][dim] device
    int nq, dim, bits, ngroups;
    int mode;                      // ScoreMode
    const uint16_t *perm0, *perm1;
    float inv_sqrt_block;
    const float *centroids;        // 2^bits
    const float *shift;            // TQ+ pair or nullptr
    const float *scale_tq;
    float level_scale;             // cs of search.rs:2815 (permute-dot only)
    // outputs
    float *q_rot;                  // [nq][dim] rotated (and TQ+-inverted) queries
    float *qscale, *qbias;         // [nq]
    uint8_t *luts;                 // [nq][lut_pitch], ngroups*32 bytes used per query (LUT modes)
    int lut_pitch;                 // bytes between the tables of consecutive queries: 32 * (ngroups rounded up to 4)
    int8_t *weights;               // [rows][dim_pad] row-major, byte d^1 = weight of coordinate d (permute-dot;
                                   // tensor-core operand: the swap matches the nibble order of a code byte)
    int dim_pad;                   // row pitch of `weights`
    uint32_t *wfrag;               // mma.sync A fragments (permute-dot), see scan kernel
    int mtiles_total;              // ceil(nq / 16)
    unsigned long long *first_invalid;  // min flat index of a query coordinate failing |x| < 1e16
};
size_t query_prep_smem_bytes(int dim);
cudaError_t launch_query_prep(const QueryPrepParams &p, cudaStream_t stream);

// ---- allow-mask utilities: bit i of little-endian u64 word i/64 <=> slot i (search.rs:2996-3004) ----
cudaError_t launch_pack_bool_mask(const uint8_t *mask_bool, int64_t n, uint64_t *words, cudaStream_t s);
cudaError_t launch_scatter_slots(const uint32_t *slots, int64_t count, uint64_t *words, cudaStream_t s);
// Clears bits >= n, counts allowed slots into *n_allowed, appends every block whose 32-bit half word is
// non-zero (search.rs:3015-3029) to live_blocks and counts them in *n_live (both zeroed by the caller).
cudaError_t launch_mask_stats(uint64_t *words, int64_t n, unsigned long long *n_allowed, uint32_t *live_blocks,
                              uint32_t *n_live, cudaStream_t s);

// ---- device copy of the id -> slot table (open addressing; keys 2^64-1 = empty, 2^64-2 = tombstone) ----
// insert: ids[i] -> slot first + i (ids not yet present).  upsert: distinct ids; slot 0xffffffff removes, else sets or inserts.
// lookup: sets the mask bit of every listed id's slot; *first_unknown = smallest list index of an id not in the table.
cudaError_t launch_idtab_insert(uint64_t *keys, uint32_t *vals, int log2cap, const uint64_t *ids, int64_t n, uint32_t first, cudaStream_t s);
cudaError_t launch_idtab_upsert(uint64_t *keys, uint32_t *vals, int log2cap, const uint64_t *ids, const uint32_t *slots, int64_t n, cudaStream_t s);
cudaError_t launch_idtab_lookup(const uint64_t *keys, const uint32_t *vals, int log2cap, const uint64_t *ids, int64_t n, uint64_t *words,
                                unsigned long long *first_unknown, cudaStream_t s);

// ---- candidate machinery ----
// Scan kernels append the key of every (query, slot) whose key is below thr[query] to
// cand[query*cap ...]; cnt[query] counts appends (it may exceed cap: the excess is dropped and the
// select kernel raises *overflow).  select merges candidates into topk[query*k ...] (ascending keys,
// kEmptyKey padded), refreshes thr and zeroes cnt.
struct CandidateBuffers {
    uint64_t *cand;
    uint32_t *cnt;
    uint64_t *thr;
    const uint64_t *lo;            // per query the lowest admissible key (paged top-k), or nullptr: every key
    uint64_t *topk;
    uint32_t *overflow;
    uint32_t *error;               // device-side wait timeouts
    int cap, k;
};
size_t select_smem_bytes(int cap, int k);
// dense_count > 0: every query has exactly that many candidates (written without counting, ScanParams::dense).
cudaError_t launch_select(const CandidateBuffers &cb, int nq, int dense_count, cudaStream_t s);
// Result keys (score-descending image << 32 | slot) of a finished search, `offset` added to every slot.
cudaError_t launch_export_keys(const uint64_t *topk, int64_t count, uint64_t offset, uint64_t *out, cudaStream_t s);
// keys[n_lists][nq][k] -> per query the k best of all lists, decoded; n_lists * k at most kMergeMaxKeys.
constexpr int kMergeMaxKeys = 8192;
// chunk_slots > 0: list r holds local slots of the shard that owns the slot chunks r, r + n_lists, ... (round-robin);
// they are turned into global slots before the merge.
cudaError_t launch_merge_keys(const uint64_t *keys, int n_lists, int nq, int k, uint32_t chunk_slots, float *scores, int64_t *slots,
                              cudaStream_t s);
// topk keys -> scores / slots with row stride k_eff = min(k, n_allowed); *k_eff_out receives it.
cudaError_t launch_finalize(const CandidateBuffers &cb, int nq, const unsigned long long *n_allowed_or_null,
                            int64_t n, float *scores, int64_t *slots, uint32_t *k_eff_out, int out_stride_is_k,
                            cudaStream_t s);

struct ScanParams {
    const uint8_t *codes;          // sequential-blocked
    const float *vec_scales;
    int64_t n;                     // vectors in the index
    int ngroups, bits;
    int mode;                      // ScoreMode
    int nq;                        // queries of this launch
    int q_base;                    // first query (offset into per-query arrays)
    const float *qscale, *qbias;
    const uint64_t *mask;          // or nullptr
    const uint32_t *live_blocks;   // or nullptr: positions are block ids
    const uint32_t *n_live;        // device count of live_blocks (when live_blocks != nullptr)
    uint32_t pos_begin, pos_end;   // positions scanned by this launch
    int dense;                     // tcgen05 scan only: write every key to cand[q][place in chunk] without counting
                                   // (the chunk holds at most cb.cap vectors; the selection is told the count)
    CandidateBuffers cb;
    // permute-dot
    const uint32_t *wfrag;
    int mtiles_total, mtile_base;
    uint32_t level_words[4];       // 16 int8 levels, entry c in byte c%4 of word c/4
    int pd_split;                  // permute-dot scan on CUDA-core MMAs: 1 = split lookup where the levels allow it
    // LUT
    const uint8_t *luts;
    int lut_pitch;                 // bytes between the tables of consecutive queries
};
// Permute-dot scan on mma.sync (int8 x int8 -> int32), up to 64 queries per launch.
cudaError_t launch_scan_pd(const ScanParams &p, int sm_count, cudaStream_t s);
// Permute-dot scan on tcgen05 tensor cores with TMEM accumulators (scan_tc.cu); all queries in one launch.
// Permute-dot: weights [rows][pitch] int8, rows % 256 == 0, pitch % 128 == 0, adjacent coordinates swapped.
// LUT families: weights = the u8 tables [rows][pitch = 32 * (ngroups rounded up to 4)], rows % 256 == 0, unused
// tables and the padding groups zero.
bool scan_tc_supported(int bits, int mode, int ngroups);
cudaError_t launch_scan_tc(const ScanParams &p, const int8_t *weights, int rows, int pitch, int sm_count,
                           int tiles_per_item, cudaStream_t s);
// The same scan for more than 256 queries with every expanded code slab shared by two query groups (scan_tc_wide.cu).
bool scan_tc_wide_supported(int bits, int mode, int ngroups, int nq_total);
cudaError_t launch_scan_tc_wide(const ScanParams &p, const int8_t *weights, int rows, int pitch, int sm_count, cudaStream_t s);
// The permute-dot scan over an int8 copy of the index (scan_tc_dense.cu): both MMA operands arrive by TMA.
// expand_blocks writes the copy: row-major int8 levels, `pitch` = expanded_pitch(dim) bytes per slot, for a range of
// 32-slot blocks or (block_list != nullptr) for the listed blocks.
bool scan_tc_dense_supported(int bits, int mode, int ngroups);
int expanded_pitch(int dim);
cudaError_t launch_expand_blocks(const uint8_t *codes, int ngroups, const uint32_t *block_list, uint32_t first_block,
                                 uint32_t n_blocks, int8_t *expanded, int pitch, const uint32_t level_words[4], int sm_count,
                                 cudaStream_t s);
cudaError_t launch_scan_tc_dense(const ScanParams &p, const int8_t *expanded, size_t exp_rows, const int8_t *weights, int rows,
                                 int pitch, int sm_count, cudaStream_t s);
// The same on CTA pairs (scan_tc_dense2.cu): tcgen05.mma.cta_group::2, each CTA loads the levels of 128 vectors and half of
// every query tile.
cudaError_t launch_scan_tc_dense_pair(const ScanParams &p, const int8_t *expanded, size_t exp_rows, const int8_t *weights, int rows,
                                      int pitch, int sm_count, cudaStream_t s);
// int8 rate (ops/s, multiply-add = 2) of back-to-back tcgen05 kind::i8 MMAs on shared-memory operands, one CTA per SM:
// the tensor-pipe roofline of the permute-dot scan on this device.  0 on failure.
double measure_int8_peak(int sm_count, double seconds, cudaStream_t s);
// Driver entry point cuTensorMapEncodeTiled (nullptr if the driver does not offer it).
void *tensor_map_encoder();
// Permute-dot scan for up to 16 queries in one launch (scan_small.cu): vectors on the M side of the warp-level MMA,
// one private bulk-copy ring per warp.  `weights` as for launch_scan_tc (row-major int8, adjacent coordinates swapped).
// variant: bits 0-1 ring depth (0: 3 stages x 3 CTAs per SM, 1: 4 x 2, 2: 6 x 2), bit 2 swizzled tensor copies.
bool scan_small_supported(const ScanParams &p, int nq_total, size_t smem_limit);
cudaError_t launch_scan_small(const ScanParams &p, const int8_t *weights, int pitch, size_t code_bytes_capacity, int variant,
                              int sm_count, size_t smem_limit, cudaStream_t s);
// LUT scan on CUDA cores.  The u8 tables of the queries of one launch sit in shared memory (32 * ngroups bytes
// each): scan_lut_width gives how many fit (4, 2, 1, or 0 when not even one does); p.nq must not exceed it.
int scan_lut_width(int ngroups, size_t smem_limit);
cudaError_t launch_scan_lut(const ScanParams &p, int sm_count, cudaStream_t s);
// lo[q] = thr[q] + 1, or the empty key when thr[q] is empty (fewer results than asked for: nothing more can follow).
cudaError_t launch_advance_floor(const uint64_t *thr, uint64_t *lo, int nq, cudaStream_t s);

}  // namespace tv
