// Tensor-memory scan over the expanded copy of the index (permute-dot family, batches of 33 queries and more).
//
// The 4-bit codes of a vector name one of 16 int8 levels per coordinate.  The scans in scan_tc.cu and scan_tc_wide.cu
// turn codes into levels in the kernel, with byte permutes that occupy the integer pipe for about as long as the MMAs
// of two query groups occupy the tensor pipe, and the two never overlap well.  The index can instead keep the levels
// themselves (`expanded`: one int8 per coordinate, row-major, row pitch = dim rounded up to 128; written by
// expand_blocks_kernel whenever rows change), twice the bytes of the codes.  Then both MMA operands arrive by TMA:
//   * warp 0 (one thread) loads, per 128-byte K slab, the A tile (128 vectors: one box, or with the compacted block list
//     of a filtered search four boxes of one 32-slot block each); warp 3 (one thread) one B tile (256 queries) per group;
//   * warps 1 and 2 (one thread each) issue the MMAs of the item's first and second query group: M = 128 vectors x
//     N = 256 queries x K = 32, tcgen05.mma kind::i8, accumulators in tensor-memory columns 256 j .. 256 j + 255;
//   * warps 4..11 are the epilogue, four per group (integer dismissal bound, then the exact float score; scan_tc_common.cuh).
// A work item is 128 vectors x 2 query groups (one group for batches up to 256 queries and for an odd last group).
// HBM traffic per item: 128 x pitch bytes of levels (read once per group pair; the pairs of a vector tile run
// together and share it in L2).  Every wait is bounded; a role whose wait runs out records the error and leaves.
#include <cuda.h>

#include <algorithm>
#include <cstddef>

#include "scan_tc_common.cuh"

namespace tv {
namespace {

constexpr int kDenseASlots = 3;
constexpr int kDenseBSlots = 5;
constexpr int kDenseBBytes = kMaxTileQueries * kSlabK;        // 32 KB: one query group, one K slab
constexpr int kDenseBlocksPerItem = 4;
constexpr int kDenseFirstEpilogueWarp = 4;
constexpr int kDenseThreads = (kDenseFirstEpilogueWarp + kEpilogueWarps) * 32;   // 384

struct DenseShared {
    uint64_t a_full[kDenseASlots];    // TMA transaction complete
    uint64_t a_empty[kDenseASlots];   // tile read by the MMAs of every group of the item (tcgen05.commit)
    uint64_t b_full[kDenseBSlots];
    uint64_t b_empty[kDenseBSlots];   // tile read by its 4 MMAs
    uint64_t d_full[2];               // accumulator half complete
    uint64_t d_empty[2];              // accumulator half drained by its 4 epilogue warps
    uint32_t tmem_base;
    uint32_t pad[3];
    float qscale[2 * kMaxTileQueries];   // per-query parameters of the item's two groups
    float qbias[2 * kMaxTileQueries];
    float qthr[2 * kMaxTileQueries];
    int ibound[2 * kMaxTileQueries];     // per query: integer sum below which no vector of the item can be a candidate
    float vs_part[2][4];                 // largest vector scale per lane quarter of the item
};
static_assert(offsetof(DenseShared, qscale) % 16 == 0, "parameter arrays must be 16-byte aligned");

__global__ void __launch_bounds__(kDenseThreads, 1)
scan_tc_dense_kernel(ScanParams p, const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap amap128,
                     const __grid_constant__ CUtensorMap wmap,
                     int n_slabs, int n_qgroups) {
    constexpr bool ONEHOT = false;
    constexpr bool fused = false;
    constexpr int kTileQueries = kMaxTileQueries;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *a_ring = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char *b_ring = a_ring + size_t(kDenseASlots) * kATileBytes;
    DenseShared *sh = reinterpret_cast<DenseShared *>(b_ring + size_t(kDenseBSlots) * kDenseBBytes);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint32_t pos_end = p.pos_end;
    if (p.live_blocks != nullptr) pos_end = min(pos_end, *p.n_live);
    const uint32_t pos_begin = min(p.pos_begin, pos_end);
    const uint32_t n_vtiles = (pos_end - pos_begin + kDenseBlocksPerItem - 1) / kDenseBlocksPerItem;
    const int n_gpairs = (n_qgroups + 1) / 2;
    const uint32_t n_items = n_vtiles * uint32_t(n_gpairs);

    if (tid == 0) {
        for (int s = 0; s < kDenseASlots; ++s) { mbar_init(&sh->a_full[s], 1); mbar_init(&sh->a_empty[s], 2); }
        for (int s = 0; s < kDenseBSlots; ++s) { mbar_init(&sh->b_full[s], 1); mbar_init(&sh->b_empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sh->d_full[b], 1); mbar_init(&sh->d_empty[b], kEpilogueWarps / 2); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = sh->tmem_base;
    // item -> (vector tile, group pair), advanced without divisions
    const uint32_t vt_step = gridDim.x / uint32_t(n_gpairs);
    const int gp_step = int(gridDim.x % uint32_t(n_gpairs));
    // groups of group pair gp: 2 gp and, unless it is the odd last one, 2 gp + 1
    auto groups_of = [&](int gp) { return 2 * gp + 1 < n_qgroups ? 2 : 1; };

    if (warp == 0) {
        // ------------------------------------------------ TMA producer of the level tiles ------------------------
        // Issuing a tensor copy costs its thread about a hundred cycles, so the level tiles and the query tiles have a
        // producer thread each.  Without a block list the four blocks of an item are neighbours: one box of 128 rows.
        if (lane == 0) {
            uint32_t it_a = 0;
            uint32_t vt = blockIdx.x / uint32_t(n_gpairs);
            int gp = int(blockIdx.x % uint32_t(n_gpairs));
            bool ok = true;
            for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                // first slot of each of the item's blocks in the expanded copy (row coordinate of its box)
                int rows[kDenseBlocksPerItem];
                int n_rows = 0;
#pragma unroll
                for (int b = 0; b < kDenseBlocksPerItem; ++b) {
                    const uint32_t pos = pos_begin + vt * kDenseBlocksPerItem + uint32_t(b);
                    rows[b] = 0;
                    if (pos < pos_end) { rows[b] = int(p.live_blocks ? p.live_blocks[pos] : pos) * 32; n_rows = b + 1; }
                }
                for (int s = 0; s < n_slabs && ok; ++s, ++it_a) {
                    const int a_slot = it_a % kDenseASlots;
                    ok = mbar_wait(&sh->a_empty[a_slot], ((it_a / kDenseASlots) & 1) ^ 1, p.cb.error);
                    if (!ok) break;
                    unsigned char *a_tile = a_ring + size_t(a_slot) * kATileBytes;
                    if (p.live_blocks == nullptr) {
                        // rows past the end of the chunk or of the copy are loaded or zero-filled alike: never read out
                        mbar_arrive_expect_tx(&sh->a_full[a_slot], uint32_t(kATileBytes));
                        tma_load_2d(a_tile, &amap128, s * kSlabK, rows[0], &sh->a_full[a_slot]);
                    } else {
                        // blocks past the end of the list are not loaded: their accumulator rows are never read out
                        mbar_arrive_expect_tx(&sh->a_full[a_slot], uint32_t(n_rows) * 32u * kSlabK);
#pragma unroll
                        for (int b = 0; b < kDenseBlocksPerItem; ++b)
                            if (b < n_rows) tma_load_2d(a_tile + b * 32 * kSlabK, &amap, s * kSlabK, rows[b], &sh->a_full[a_slot]);
                    }
                }
                vt += vt_step; gp += gp_step;
                if (gp >= n_gpairs) { gp -= n_gpairs; ++vt; }
            }
        }
    } else if (warp == 3) {
        // ------------------------------------------------ TMA producer of the query tiles, group by group -----------
        if (lane == 0) {
            uint32_t it_b = 0;
            int gp = int(blockIdx.x % uint32_t(n_gpairs));
            bool ok = true;
            for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                const int gcount = groups_of(gp);
                for (int s = 0; s < n_slabs && ok; ++s) {
                    for (int j = 0; j < gcount && ok; ++j, ++it_b) {
                        const int slot = it_b % kDenseBSlots;
                        ok = mbar_wait(&sh->b_empty[slot], ((it_b / kDenseBSlots) & 1) ^ 1, p.cb.error);
                        if (!ok) break;
                        mbar_arrive_expect_tx(&sh->b_full[slot], kDenseBBytes);
                        tma_load_2d(b_ring + size_t(slot) * kDenseBBytes, &wmap, s * kSlabK, (2 * gp + j) * kTileQueries, &sh->b_full[slot]);
                    }
                }
                gp += gp_step;
                if (gp >= n_gpairs) gp -= n_gpairs;
            }
        }
    } else if (warp == 1 || warp == 2) {
        // ------------------------------------------------ MMA issuers: warp 1 for group 0, warp 2 for group 1 --------
        // One thread per group: waiting on a barrier and issuing four MMAs each take a few hundred cycles of the
        // issuing thread, about what the four MMAs take to run.  The two groups write different tensor-memory columns,
        // so their MMAs need no order between them.
        if (lane == 0) {
            const int j = warp - 1;                            // this issuer's group within every item
            uint32_t it_a = 0, b_base = 0, uses = 0;
            int gp = int(blockIdx.x % uint32_t(n_gpairs));
            bool ok = true;
            for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                const int gcount = groups_of(gp);
                if (j < gcount) {
                    for (int s = 0; s < n_slabs && ok; ++s) {
                        const uint32_t ia = it_a + uint32_t(s);
                        const int a_slot = ia % kDenseASlots;
                        if (s == 0) {                         // the half must have been drained by the previous item's epilogue
                            ok = mbar_wait(&sh->d_empty[j], (uses & 1) ^ 1, p.cb.error);
                            if (!ok) break;
                        }
                        ok = mbar_wait(&sh->a_full[a_slot], (ia / kDenseASlots) & 1, p.cb.error);
                        if (!ok) break;
                        const uint32_t ib = b_base + uint32_t(s * gcount + j);
                        const int b_slot = ib % kDenseBSlots;
                        ok = mbar_wait(&sh->b_full[b_slot], (ib / kDenseBSlots) & 1, p.cb.error);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t a_addr = smem_u32(a_ring + size_t(a_slot) * kATileBytes);
                        const uint32_t b_addr = smem_u32(b_ring + size_t(b_slot) * kDenseBBytes);
                        const uint32_t d_tmem = tmem_base + uint32_t(j) * kTileQueries;
#pragma unroll
                        for (int k = 0; k < kSlabK / 32; ++k)
                            umma_i8<kTileQueries>(d_tmem, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), (s | k) != 0);
                        umma_commit(&sh->b_empty[b_slot]);
                        umma_commit(&sh->a_empty[a_slot]);    // the tile is free once both groups have read it
                        if (gcount == 1) umma_commit(&sh->a_empty[a_slot]);   // an item of one group: its issuer signs twice
                        if (s == n_slabs - 1) { umma_commit(&sh->d_full[j]); ++uses; }
                    }
                }
                it_a += uint32_t(n_slabs);
                b_base += uint32_t(n_slabs * gcount);
                gp += gp_step;
                if (gp >= n_gpairs) gp -= n_gpairs;
            }
        }
    } else if (warp >= kDenseFirstEpilogueWarp) {
        // ------------------------------------------------ epilogue: warps of half j drain group j of the item ----
        const int quarter = warp & 3;                     // TMEM lanes 32*quarter .. +31 are this warp's
        const int half = (warp - kDenseFirstEpilogueWarp) >> 2;                 // which group of the item
        const int ht = ((warp - kDenseFirstEpilogueWarp) & 3) * 32 + lane;      // 0..127 among the threads of this half
        uint32_t used = 0;                                // items in which this half took part
        uint32_t vt = blockIdx.x / uint32_t(n_gpairs);
        int gp = int(blockIdx.x % uint32_t(n_gpairs));
        bool ok = true;
        float *qscale = sh->qscale + half * kTileQueries, *qbias = sh->qbias + half * kTileQueries, *qthr = sh->qthr + half * kTileQueries;
        for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            if (half < groups_of(gp)) {
                const int qg = 2 * gp + half;
                // this lane's vector, and the largest vector scale of the item (dismissal_bound)
                const int row = quarter * 32 + lane;                     // vector within the item
                const uint32_t pos = pos_begin + vt * kDenseBlocksPerItem + uint32_t(row >> 5);
                const bool have_row = pos < pos_end;
                uint32_t blk = 0;
                if (have_row) blk = p.live_blocks ? p.live_blocks[pos] : pos;
                const int64_t slot = int64_t(blk) * 32 + (row & 31);
                bool live = have_row && slot < p.n;
                if (live && p.mask) live = (p.mask[slot >> 6] >> (slot & 63)) & 1ull;
                const float vs = live ? p.vec_scales[slot] : 0.0f;
                {
                    float m = vs;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(kFullMask, m, o));
                    if (lane == 0) sh->vs_part[half][quarter] = m;
                }
                asm volatile("bar.sync %0, %1;" ::"r"(1 + half), "r"(128) : "memory");
                const float vs_max = fmaxf(fmaxf(sh->vs_part[half][0], sh->vs_part[half][1]), fmaxf(sh->vs_part[half][2], sh->vs_part[half][3]));
                // per-query parameters of this group: two queries per thread of the half
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int c = ht + 128 * e, ql = qg * kTileQueries + c;
                    float qs = 0.f, qb = 0.f, th = INFINITY;
                    if (ql < p.q_base + p.nq) {
                        qs = p.qscale[ql]; qb = p.qbias[ql];
                        const uint64_t key = p.cb.thr[ql];
                        th = key == kEmptyKey ? -INFINITY : desc_bits_to_score(uint32_t(key >> 32));
                    }
                    qscale[c] = qs; qbias[c] = qb; qthr[c] = th;
                    sh->ibound[half * kTileQueries + c] = dismissal_bound(qs, qb, th, vs_max);
                }
                asm volatile("bar.sync %0, %1;" ::"r"(1 + half), "r"(128) : "memory");

                // warp-uniform outcome; a warp whose wait ran out still meets the others at the barrier below
                ok = __all_sync(kFullMask, mbar_wait(&sh->d_full[half], used & 1, p.cb.error));
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(half) * kTileQueries;
                for (int c0 = 0; c0 < (ok ? kTileQueries : 0); c0 += 32) {
                    uint32_t acc[32];
                    tmem_ld32(taddr + c0, acc);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (p.dense) {
                        // first chunk of a search: every vector's key goes to the list position of its place in the chunk
                        const uint32_t at = (vt * kDenseBlocksPerItem) * 32u + uint32_t(row);
                        if (have_row)
                            write_piece<ONEHOT>(acc, qscale + c0, qbias + c0, fused, vs, live, slot, qg * kTileQueries + c0, p.q_base + p.nq, at, p.cb);
                        continue;
                    }
                    sift_piece<ONEHOT>(acc, sh->ibound + half * kTileQueries + c0, qscale + c0, qbias + c0, qthr + c0, fused, vs, live, slot,
                                       qg * kTileQueries + c0, taddr + c0, p.cb);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->d_empty[half]);
                // the parameters are rewritten for the next item only after every warp of the half is done with them
                asm volatile("bar.sync %0, %1;" ::"r"(1 + half), "r"(128) : "memory");
                ++used;
                if (!ok) break;
            }
            vt += vt_step; gp += gp_step;
            if (gp >= n_gpairs) { gp -= n_gpairs; ++vt; }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// Levels of 32-slot blocks: expanded[slot][2 g] = level[low nibble of code byte g], [2 g + 1] = level[high nibble]
// (the order in which query preparation lays out the int8 query weights).  One CTA per block and pass; a warp takes
// 4 byte-groups x 32 slots per step (one 128-byte line of codes), turns them in registers and writes, per slot, the
// 8 levels of those groups; shared memory gathers them so that every slot's row is written in runs of 128 bytes.
constexpr int kExpandThreads = 256;
__global__ void __launch_bounds__(kExpandThreads)
expand_blocks_kernel(const uint8_t *codes, int ngroups, const uint32_t *block_list, uint32_t first_block, uint32_t n_blocks,
                     int8_t *expanded, int pitch, uint4 level_words) {
    __shared__ __align__(16) uint8_t tile[32][128 + 16];      // 32 slots x 64 groups x 2 levels; rows padded against bank conflicts
    __shared__ uint8_t lv[16];
    const int tid = threadIdx.x;
    if (tid < 16) {
        const uint32_t w = tid < 4 ? level_words.x : (tid < 8 ? level_words.y : (tid < 12 ? level_words.z : level_words.w));
        lv[tid] = uint8_t(w >> ((tid & 3) * 8));
    }
    __syncthreads();
    for (uint32_t b = blockIdx.x; b < n_blocks; b += gridDim.x) {
        const uint32_t blk = block_list ? block_list[b] : first_block + b;
        const uint8_t *src = codes + size_t(blk) * ngroups * 32;
        int8_t *dst = expanded + size_t(blk) * 32 * pitch;
        for (int g0 = 0; g0 < ngroups; g0 += 64) {
            const int gn = min(64, ngroups - g0);
            // thread: word column c (4 slots) of group rows r, r + 32
            for (int i = tid; i < gn * 8; i += kExpandThreads) {
                const int r = i >> 3, c = i & 7;
                const uint32_t w = __ldg(reinterpret_cast<const uint32_t *>(src + size_t(g0 + r) * 32) + c);
                // byte j of w = code byte of slot 4c + j; its two nibbles -> two levels
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t byte = (w >> (8 * j)) & 0xffu;
                    const uint32_t lv_lo = lv[byte & 15u], lv_hi = lv[byte >> 4];
                    *reinterpret_cast<uint16_t *>(&tile[4 * c + j][2 * r]) = uint16_t(lv_lo | (lv_hi << 8));
                }
            }
            __syncthreads();
            // 32 rows x (2 gn) bytes, written 16 bytes per thread
            const int chunks = (2 * gn) / 16;                 // gn is a multiple of 4 (permute-dot geometry): whole 8-byte runs
            for (int i = tid; i < 32 * 8; i += kExpandThreads) {
                const int row = i >> 3, ch = i & 7;
                if (ch < chunks)
                    *reinterpret_cast<uint4 *>(dst + size_t(row) * pitch + 2 * g0 + ch * 16) = *reinterpret_cast<const uint4 *>(&tile[row][ch * 16]);
                else if (ch == chunks && (2 * gn) % 16)
                    *reinterpret_cast<uint2 *>(dst + size_t(row) * pitch + 2 * g0 + ch * 16) = *reinterpret_cast<const uint2 *>(&tile[row][ch * 16]);
            }
            __syncthreads();
        }
    }
}

}  // namespace

bool scan_tc_dense_supported(int bits, int mode, int ngroups) {
    return mode == kModePermuteDot && scan_tc_supported(bits, mode, ngroups);
}

// Row pitch of the expanded copy: whole K slabs.
int expanded_pitch(int dim) { return (dim + kSlabK - 1) / kSlabK * kSlabK; }

cudaError_t launch_expand_blocks(const uint8_t *codes, int ngroups, const uint32_t *block_list, uint32_t first_block,
                                 uint32_t n_blocks, int8_t *expanded, int pitch, const uint32_t level_words[4], int sm_count,
                                 cudaStream_t s) {
    if (n_blocks == 0) return cudaSuccess;
    const unsigned grid = unsigned(std::min<uint64_t>(n_blocks, uint64_t(sm_count) * 8));
    expand_blocks_kernel<<<grid, kExpandThreads, 0, s>>>(codes, ngroups, block_list, first_block, n_blocks, expanded, pitch,
                                                          make_uint4(level_words[0], level_words[1], level_words[2], level_words[3]));
    return cudaGetLastError();
}

// expanded / exp_rows: the expanded copy and the number of rows it was allocated for (a multiple of 32).
// weights / pitch / rows as for launch_scan_tc; pitch must equal the row pitch of the expanded copy.
cudaError_t launch_scan_tc_dense(const ScanParams &p, const int8_t *expanded, size_t exp_rows, const int8_t *weights, int rows,
                                 int pitch, int sm_count, cudaStream_t s) {
    if (p.nq <= 0 || p.pos_end <= p.pos_begin) return cudaSuccess;
    typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                      const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(tensor_map_encoder());
    if (!enc) return cudaErrorNotSupported;
    const int nq_all = p.q_base + p.nq;
    CUtensorMap wmap, amap, amap128;
    const cuuint64_t strides[1] = {cuuint64_t(pitch)};
    const cuuint32_t estr[2] = {1, 1};
    {
        const cuuint64_t dims[2] = {cuuint64_t(pitch), cuuint64_t(rows)};
        const cuuint32_t box[2] = {cuuint32_t(kSlabK), cuuint32_t(kMaxTileQueries)};
        if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t *>(weights), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    {
        const cuuint64_t dims[2] = {cuuint64_t(pitch), cuuint64_t(exp_rows)};
        const cuuint32_t box[2] = {cuuint32_t(kSlabK), 32u};
        if (enc(&amap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t *>(expanded), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
        const cuuint32_t box128[2] = {cuuint32_t(kSlabK), cuuint32_t(kMmaM)};
        if (enc(&amap128, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t *>(expanded), dims, strides, box128, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    const int n_slabs = pitch / kSlabK;
    const int n_qgroups = (nq_all + kMaxTileQueries - 1) / kMaxTileQueries;
    const int n_gpairs = (n_qgroups + 1) / 2;
    const size_t smem = size_t(kDenseASlots) * kATileBytes + size_t(kDenseBSlots) * kDenseBBytes + sizeof(DenseShared) + 1024;
    const uint32_t vtiles = (p.pos_end - p.pos_begin + kDenseBlocksPerItem - 1) / kDenseBlocksPerItem;
    const uint64_t items = uint64_t(vtiles) * n_gpairs;
    // a multiple of the group-pair count keeps the CTAs that share a vector tile in step (levels hit L2)
    unsigned grid = unsigned(sm_count - sm_count % n_gpairs);
    if (grid == 0) grid = unsigned(sm_count);
    if (items < grid) grid = unsigned(items);
    cudaError_t e = cudaFuncSetAttribute(scan_tc_dense_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
    scan_tc_dense_kernel<<<grid, kDenseThreads, smem, s>>>(p, amap, amap128, wmap, n_slabs, n_qgroups);
    return cudaGetLastError();
}

}  // namespace tv
