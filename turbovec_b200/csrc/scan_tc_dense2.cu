// The dense tensor-memory scan (scan_tc_dense.cu) on CTA pairs: tcgen05.mma.cta_group::2, M = 256 across two SMs.
//
// In the one-CTA kernel every SM pulls, per 128-byte K slab, its 16 KB tile of levels and 32 KB of query weights per
// query group through L2: 80 KB per 1,030 tensor-pipe cycles with two groups, which is what the L2-to-SM fabric
// delivers at best.  Here a work item is 256 vectors x 2 query groups, run by a cluster of two CTAs:
//   * each CTA loads the level tile of ITS 128 vectors and ONE HALF (128 queries) of each group's query tile; the MMAs
//     of the pair read both halves, so an SM pulls 48 KB per slab for the same multiply-adds;
//   * the even CTA (the leader) issues the MMAs for both, one thread per query group; each CTA's 128 x 256 accumulator
//     tiles land in its own tensor memory and are drained by its own epilogue warps.
// Barriers: `a_full`, `b_full` and `d_empty` live in the leader and collect both CTAs (TMA transactions addressed to the
// leader's barrier, remote arrivals); `a_empty`, `b_empty` and `d_full` exist in both CTAs and the leader commits to
// each.  No load is multicast.  Every wait is bounded; a role whose wait runs out records the error and leaves its
// loop, and both CTAs always meet at the closing cluster barrier.
#include <cuda.h>

#include <algorithm>
#include <cstddef>

#include "scan_tc_common.cuh"

namespace tv {
namespace {

constexpr int kASlots = 4;
constexpr int kBSlots = 8;
constexpr int kBHalfBytes = 128 * kSlabK;                     // this CTA's half of one group's query tile: 16 KB
constexpr int kBlocksPerCta = 4;
constexpr int kFirstEpilogueWarp = 4;
constexpr int kPairThreads = (kFirstEpilogueWarp + kEpilogueWarps) * 32;   // 384

struct DensePairShared {
    uint64_t a_full[kASlots];         // leader's copy: both CTAs' level tiles have landed
    uint64_t a_empty[kASlots];        // per CTA: tile read by the MMAs of every group of the item
    uint64_t b_full[kBSlots];         // leader's copy: both halves of a query tile have landed
    uint64_t b_empty[kBSlots];        // per CTA
    uint64_t d_full[2];               // per CTA: accumulator half complete
    uint64_t d_empty[2];              // leader's copy: drained by the 4 epilogue warps of the half in both CTAs
    uint32_t tmem_base;
    uint32_t pad[3];
    float qscale[2 * kMaxTileQueries];
    float qbias[2 * kMaxTileQueries];
    float qthr[2 * kMaxTileQueries];
    int ibound[2 * kMaxTileQueries];
    float vs_part[2][4];
};
static_assert(offsetof(DensePairShared, qscale) % 16 == 0, "parameter arrays must be 16-byte aligned");

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
scan_tc_dense_pair_kernel(ScanParams p, const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap amap128,
                          const __grid_constant__ CUtensorMap wmap, int n_slabs, int n_qgroups) {
    constexpr bool ONEHOT = false;
    constexpr bool fused = false;
    constexpr int kTileQueries = kMaxTileQueries;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *a_ring = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char *b_ring = a_ring + size_t(kASlots) * kATileBytes;
    DensePairShared *sh = reinterpret_cast<DensePairShared *>(b_ring + size_t(kBSlots) * kBHalfBytes);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_ctarank();                  // 0 = leader
    const uint32_t cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    uint32_t pos_end = p.pos_end;
    if (p.live_blocks != nullptr) pos_end = min(pos_end, *p.n_live);
    const uint32_t pos_begin = min(p.pos_begin, pos_end);
    const uint32_t n_vtiles = (pos_end - pos_begin + 2 * kBlocksPerCta - 1) / (2 * kBlocksPerCta);   // tiles of 256 vectors
    const int n_gpairs = (n_qgroups + 1) / 2;
    const uint32_t n_items = n_vtiles * uint32_t(n_gpairs);

    if (tid == 0) {
        for (int s = 0; s < kASlots; ++s) { mbar_init(&sh->a_full[s], 2); mbar_init(&sh->a_empty[s], 2); }
        for (int s = 0; s < kBSlots; ++s) { mbar_init(&sh->b_full[s], 2); mbar_init(&sh->b_empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sh->d_full[b], 1); mbar_init(&sh->d_empty[b], kEpilogueWarps); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                                          // one warp of each CTA, the same one in both
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync_all();                                       // barriers initialised and TMEM allocated in both CTAs
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = sh->tmem_base;
    // item -> (vector tile, group pair), advanced without divisions
    const uint32_t vt_step = n_clusters / uint32_t(n_gpairs);
    const int gp_step = int(n_clusters % uint32_t(n_gpairs));
    auto groups_of = [&](int gp) { return 2 * gp + 1 < n_qgroups ? 2 : 1; };

    if (warp == 0) {
        // ------------------------------------------------ TMA producer: the level tile of this CTA's 128 vectors ----
        if (lane == 0) {
            uint32_t it_a = 0;
            uint32_t vt = cluster_id / uint32_t(n_gpairs);
            int gp = int(cluster_id % uint32_t(n_gpairs));
            bool ok = true;
            for (uint32_t item = cluster_id; item < n_items && ok; item += n_clusters) {
                int rows[kBlocksPerCta];
                int n_rows = 0;
#pragma unroll
                for (int b = 0; b < kBlocksPerCta; ++b) {
                    const uint32_t pos = pos_begin + (vt * 2 + rank) * kBlocksPerCta + uint32_t(b);
                    rows[b] = 0;
                    if (pos < pos_end) { rows[b] = int(p.live_blocks ? p.live_blocks[pos] : pos) * 32; n_rows = b + 1; }
                }
                // without a block list the tile is one box; its row may lie past the chunk (rank 1 of an odd last tile)
                const int row0 = int(pos_begin + (vt * 2 + rank) * kBlocksPerCta) * 32;
                for (int s = 0; s < n_slabs && ok; ++s, ++it_a) {
                    const int a_slot = it_a % kASlots;
                    ok = mbar_wait(&sh->a_empty[a_slot], ((it_a / kASlots) & 1) ^ 1, p.cb.error);
                    if (!ok) break;
                    const uint32_t leader_full = map_to_cta(smem_u32(&sh->a_full[a_slot]), 0);
                    unsigned char *a_tile = a_ring + size_t(a_slot) * kATileBytes;
                    if (p.live_blocks == nullptr) {
                        mbar_arrive_expect_tx_cluster(leader_full, uint32_t(kATileBytes));
                        tma_load_2d_pair(a_tile, &amap128, s * kSlabK, row0, leader_full);
                    } else {
                        mbar_arrive_expect_tx_cluster(leader_full, uint32_t(n_rows) * 32u * kSlabK);
#pragma unroll
                        for (int b = 0; b < kBlocksPerCta; ++b)
                            if (b < n_rows) tma_load_2d_pair(a_tile + b * 32 * kSlabK, &amap, s * kSlabK, rows[b], leader_full);
                    }
                }
                vt += vt_step; gp += gp_step;
                if (gp >= n_gpairs) { gp -= n_gpairs; ++vt; }
            }
        }
    } else if (warp == 3) {
        // ------------------------------------------------ TMA producer: this CTA's half of every query tile ---------
        if (lane == 0) {
            uint32_t it_b = 0;
            int gp = int(cluster_id % uint32_t(n_gpairs));
            bool ok = true;
            for (uint32_t item = cluster_id; item < n_items && ok; item += n_clusters) {
                const int gcount = groups_of(gp);
                for (int s = 0; s < n_slabs && ok; ++s) {
                    for (int j = 0; j < gcount && ok; ++j, ++it_b) {
                        const int slot = it_b % kBSlots;
                        ok = mbar_wait(&sh->b_empty[slot], ((it_b / kBSlots) & 1) ^ 1, p.cb.error);
                        if (!ok) break;
                        const uint32_t leader_full = map_to_cta(smem_u32(&sh->b_full[slot]), 0);
                        mbar_arrive_expect_tx_cluster(leader_full, kBHalfBytes);
                        tma_load_2d_pair(b_ring + size_t(slot) * kBHalfBytes, &wmap, s * kSlabK,
                                         (2 * gp + j) * kTileQueries + int(rank) * 128, leader_full);
                    }
                }
                gp += gp_step;
                if (gp >= n_gpairs) gp -= n_gpairs;
            }
        }
    } else if (warp == 1 || warp == 2) {
        // ------------------------------------------------ MMA issuers of the leader: warp 1 group 0, warp 2 group 1 ----
        if (lane == 0 && rank == 0) {
            const int j = warp - 1;
            uint32_t it_a = 0, b_base = 0, uses = 0;
            int gp = int(cluster_id % uint32_t(n_gpairs));
            bool ok = true;
            for (uint32_t item = cluster_id; item < n_items && ok; item += n_clusters) {
                const int gcount = groups_of(gp);
                if (j < gcount) {
                    for (int s = 0; s < n_slabs && ok; ++s) {
                        const uint32_t ia = it_a + uint32_t(s);
                        const int a_slot = ia % kASlots;
                        if (s == 0) {                         // the half must have been drained in both CTAs
                            ok = mbar_wait(&sh->d_empty[j], (uses & 1) ^ 1, p.cb.error);
                            if (!ok) break;
                        }
                        ok = mbar_wait(&sh->a_full[a_slot], (ia / kASlots) & 1, p.cb.error);
                        if (!ok) break;
                        const uint32_t ib = b_base + uint32_t(s * gcount + j);
                        const int b_slot = ib % kBSlots;
                        ok = mbar_wait(&sh->b_full[b_slot], (ib / kBSlots) & 1, p.cb.error);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t a_addr = smem_u32(a_ring + size_t(a_slot) * kATileBytes);
                        const uint32_t b_addr = smem_u32(b_ring + size_t(b_slot) * kBHalfBytes);
                        const uint32_t d_tmem = tmem_base + uint32_t(j) * kTileQueries;
#pragma unroll
                        for (int k = 0; k < kSlabK / 32; ++k)
                            umma_i8_pair(d_tmem, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), (s | k) != 0);
                        // the tiles may be refilled in both CTAs once these MMAs have read them
                        const uint32_t be = smem_u32(&sh->b_empty[b_slot]), ae = smem_u32(&sh->a_empty[a_slot]);
                        umma_commit_pair(be);
                        umma_commit_pair(map_to_cta(be, 1));
                        const int signs = gcount == 1 ? 2 : 1;         // an item of one group: its issuer signs for both
                        for (int r = 0; r < signs; ++r) {
                            umma_commit_pair(ae);
                            umma_commit_pair(map_to_cta(ae, 1));
                        }
                        if (s == n_slabs - 1) {
                            const uint32_t f = smem_u32(&sh->d_full[j]);
                            umma_commit_pair(f);
                            umma_commit_pair(map_to_cta(f, 1));
                            ++uses;
                        }
                    }
                }
                it_a += uint32_t(n_slabs);
                b_base += uint32_t(n_slabs * gcount);
                gp += gp_step;
                if (gp >= n_gpairs) gp -= n_gpairs;
            }
        }
    } else if (warp >= kFirstEpilogueWarp) {
        // ------------------------------------------------ epilogue: warps of half j drain group j of the item ----
        const int quarter = warp & 3;                     // TMEM lanes 32*quarter .. +31 are this warp's
        const int half = (warp - kFirstEpilogueWarp) >> 2;                 // which group of the item
        const int ht = ((warp - kFirstEpilogueWarp) & 3) * 32 + lane;      // 0..127 among the threads of this half
        uint32_t used = 0;                                // items in which this half took part
        uint32_t vt = cluster_id / uint32_t(n_gpairs);
        int gp = int(cluster_id % uint32_t(n_gpairs));
        bool ok = true;
        float *qscale = sh->qscale + half * kTileQueries, *qbias = sh->qbias + half * kTileQueries, *qthr = sh->qthr + half * kTileQueries;
        for (uint32_t item = cluster_id; item < n_items && ok; item += n_clusters) {
            if (half < groups_of(gp)) {
                const int qg = 2 * gp + half;
                // this lane's vector, and the largest vector scale of the item (dismissal_bound)
                const int row = quarter * 32 + lane;                     // vector within the item
                const uint32_t pos = pos_begin + (vt * 2 + rank) * kBlocksPerCta + uint32_t(row >> 5);
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
                const float4 *ps = reinterpret_cast<const float4 *>(qscale);
                const float4 *pbias = reinterpret_cast<const float4 *>(qbias);
                const float4 *pt = reinterpret_cast<const float4 *>(qthr);
                const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(half) * kTileQueries;
                for (int c0 = 0; c0 < (ok ? kTileQueries : 0); c0 += 32) {
                    uint32_t acc[32];
                    tmem_ld32(taddr + c0, acc);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (p.dense) {
                        // first chunk of a search: every vector's key goes to the list position of its place in the chunk
                        const uint32_t at = ((vt * 2 + rank) * kBlocksPerCta) * 32u + uint32_t(row);
                        if (have_row) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const int c = c0 + j;
                                const int ql = qg * kTileQueries + c;
                                if (ql < p.q_base + p.nq) {
                                    const float score = final_score<ONEHOT>(fused, acc[j], qscale[c], qbias[c], vs);
                                    p.cb.cand[size_t(ql) * p.cb.cap + at] = live ? make_key(score, uint32_t(slot)) : kEmptyKey;
                                }
                            }
                        }
                        continue;
                    }
                    // one integer compare per column dismisses the piece unless some column could be a candidate
                    {
                        const int4 *pi = reinterpret_cast<const int4 *>(sh->ibound + half * kTileQueries + c0);
                        bool may = false;
#pragma unroll
                        for (int j4 = 0; j4 < 8; ++j4) {
                            const int4 b = pi[j4];
                            may |= int(acc[4 * j4 + 0]) >= b.x;
                            may |= int(acc[4 * j4 + 1]) >= b.y;
                            may |= int(acc[4 * j4 + 2]) >= b.z;
                            may |= int(acc[4 * j4 + 3]) >= b.w;
                        }
                        if (!__any_sync(kFullMask, may && live)) continue;
                    }
                    bool any = false;
#pragma unroll
                    for (int j4 = 0; j4 < 8; ++j4) {
                        const float4 s4 = ps[(c0 >> 2) + j4], b4 = pbias[(c0 >> 2) + j4], t4 = pt[(c0 >> 2) + j4];
                        any |= final_score<ONEHOT>(fused, acc[4 * j4 + 0], s4.x, b4.x, vs) >= t4.x;
                        any |= final_score<ONEHOT>(fused, acc[4 * j4 + 1], s4.y, b4.y, vs) >= t4.y;
                        any |= final_score<ONEHOT>(fused, acc[4 * j4 + 2], s4.z, b4.z, vs) >= t4.z;
                        any |= final_score<ONEHOT>(fused, acc[4 * j4 + 3], s4.w, b4.w, vs) >= t4.w;
                    }
                    any = any && live;
                    if (__any_sync(kFullMask, any)) {          // rare, warp-uniform: re-read in pieces of 8 and append
#pragma unroll 1
                        for (int c1 = 0; c1 < 32; c1 += 8) {
                            uint32_t a8[8];
                            tmem_ld8(taddr + c0 + c1, a8);
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                            if (any) {
#pragma unroll
                                for (int e = 0; e < 8; ++e) {
                                    const int c = c0 + c1 + e;
                                    const float score = final_score<ONEHOT>(fused, a8[e], qscale[c], qbias[c], vs);
                                    if (score >= qthr[c]) {
                                        const int ql = qg * kTileQueries + c;
                                        const uint64_t key = make_key(score, uint32_t(slot));
                                        if (key < p.cb.thr[ql] && (p.cb.lo == nullptr || key >= p.cb.lo[ql])) {
                                            const uint32_t at = atomicAdd(&p.cb.cnt[ql], 1u);
                                            if (at < uint32_t(p.cb.cap)) p.cb.cand[size_t(ql) * p.cb.cap + at] = key;
                                        }
                                    }
                                }
                            }
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&sh->d_empty[half]), 0));   // the leader's barrier counts both CTAs
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
    cluster_sync_all();                                       // neither CTA leaves while the other may still reach into it
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

}  // namespace

// Arguments as for launch_scan_tc_dense.
cudaError_t launch_scan_tc_dense_pair(const ScanParams &p, const int8_t *expanded, size_t exp_rows, const int8_t *weights, int rows,
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
    auto encode = [&](CUtensorMap *m, const int8_t *base, size_t n_rows, uint32_t box_rows) {
        const cuuint64_t dims[2] = {cuuint64_t(pitch), cuuint64_t(n_rows)};
        const cuuint32_t box[2] = {cuuint32_t(kSlabK), box_rows};
        return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    };
    if (!encode(&wmap, weights, size_t(rows), 128u) || !encode(&amap, expanded, exp_rows, 32u) || !encode(&amap128, expanded, exp_rows, 128u))
        return cudaErrorInvalidValue;
    const int n_slabs = pitch / kSlabK;
    const int n_qgroups = (nq_all + kMaxTileQueries - 1) / kMaxTileQueries;
    const int n_gpairs = (n_qgroups + 1) / 2;
    const size_t smem = size_t(kASlots) * kATileBytes + size_t(kBSlots) * kBHalfBytes + sizeof(DensePairShared) + 1024;
    const uint32_t vtiles = (p.pos_end - p.pos_begin + 2 * kBlocksPerCta - 1) / (2 * kBlocksPerCta);
    const uint64_t items = uint64_t(vtiles) * n_gpairs;
    // clusters of two CTAs; a multiple of the group-pair count keeps the clusters that share a vector tile in step
    unsigned clusters = unsigned(sm_count / 2);
    clusters -= clusters % unsigned(n_gpairs);
    if (clusters == 0) clusters = unsigned(sm_count / 2);
    if (items < clusters) clusters = unsigned(items);
    cudaError_t e = cudaFuncSetAttribute(scan_tc_dense_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
    scan_tc_dense_pair_kernel<<<clusters * 2, kPairThreads, smem, s>>>(p, amap, amap128, wmap, n_slabs, n_qgroups);
    return cudaGetLastError();
}

}  // namespace tv
