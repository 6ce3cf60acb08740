// The dense tensor-memory scan (scan_tc_dense.cu) on CTA pairs: tcgen05.mma.cta_group::2, M = 256 across two SMs.
//
// In the one-CTA kernel a work item keeps both halves of tensor memory busy (two query groups), so the tensor pipe
// idles while the epilogue drains them, and every SM pulls 80 KB per 128-byte K slab through L2.  Here a work item is
// 256 vectors x ONE query group, run by a cluster of two CTAs:
//   * each CTA loads the level tile of ITS 128 vectors and ONE HALF (128 queries) of the query tile: 32 KB per slab and
//     SM; the MMAs of the pair read both halves;
//   * the even CTA (the leader) issues the MMAs for both; each CTA's 128 x 256 accumulator tile lands in its own tensor
//     memory, in one of two buffers, so the MMAs of the next item run while the epilogue warps drain this one.
// Items that share a vector tile (the query groups of a batch) run at the same time on neighbouring clusters and share
// the level tile in L2.
// Barriers: `full` and `d_empty` live in the leader and collect both CTAs (TMA transactions addressed to the leader's
// barrier, remote arrivals); `empty` and `d_full` exist in both CTAs and the leader commits to each.  No load is
// multicast.  Every wait is bounded; a role whose wait runs out records the error and leaves its loop, and both CTAs
// always meet at the closing cluster barrier.
#include <cuda.h>

#include <algorithm>
#include <cstddef>

#include "scan_tc_common.cuh"

namespace tv {
namespace {

constexpr int kStages = 6;
constexpr int kBHalfBytes = 128 * kSlabK;                     // this CTA's half of the query tile: 16 KB
constexpr int kStageBytes = kATileBytes + kBHalfBytes;        // 32 KB
constexpr int kBlocksPerCta = 4;
constexpr int kFirstEpilogueWarp = 4;
constexpr int kPairThreads = (kFirstEpilogueWarp + kEpilogueWarps) * 32;   // 384

struct DensePairShared {
    uint64_t full[kStages];           // leader's copy: both CTAs' tiles of the stage have landed
    uint64_t empty[kStages];          // per CTA: stage read by the pair's MMAs
    uint64_t d_full[2];               // per CTA: accumulator buffer complete
    uint64_t d_empty[2];              // leader's copy: buffer drained by the 8 epilogue warps of both CTAs
    uint32_t tmem_base;
    uint32_t epilogue_failed;         // a wait of some epilogue warp ran out: all of them leave after the item
    uint32_t pad[2];
    float qscale[kMaxTileQueries];    // per-query parameters of the item's group
    float qbias[kMaxTileQueries];
    float qthr[kMaxTileQueries];
    int ibound[kMaxTileQueries];      // per query: integer sum below which no vector of the item can be a candidate
    float vs_part[2][4];              // largest vector scale per lane quarter (written by both column halves)
};
static_assert(offsetof(DensePairShared, qscale) % 16 == 0, "parameter arrays must be 16-byte aligned");

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
scan_tc_dense_pair_kernel(ScanParams p, const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap amap128,
                          const __grid_constant__ CUtensorMap wmap, int n_slabs, int n_qgroups) {
    constexpr bool ONEHOT = false;
    constexpr bool fused = false;
    constexpr int kTileQueries = kMaxTileQueries;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *stages = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    DensePairShared *sh = reinterpret_cast<DensePairShared *>(stages + size_t(kStages) * kStageBytes);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_ctarank();                  // 0 = leader
    const uint32_t cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    uint32_t pos_end = p.pos_end;
    if (p.live_blocks != nullptr) pos_end = min(pos_end, *p.n_live);
    const uint32_t pos_begin = min(p.pos_begin, pos_end);
    const uint32_t n_vtiles = (pos_end - pos_begin + 2 * kBlocksPerCta - 1) / (2 * kBlocksPerCta);   // tiles of 256 vectors
    const uint32_t n_items = n_vtiles * uint32_t(n_qgroups);

    if (tid == 0) {
        sh->epilogue_failed = 0;
        for (int s = 0; s < kStages; ++s) { mbar_init(&sh->full[s], 2); mbar_init(&sh->empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sh->d_full[b], 1); mbar_init(&sh->d_empty[b], 2 * kEpilogueWarps); }
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
    // item -> (vector tile, query group), advanced without divisions
    const uint32_t vt_step = n_clusters / uint32_t(n_qgroups);
    const int qg_step = int(n_clusters % uint32_t(n_qgroups));

    if (warp == 0) {
        // ------------------------------------------------ TMA producer: this CTA's level tile and query half-tile ----
        if (lane == 0) {
            uint32_t it = 0;
            uint32_t vt = cluster_id / uint32_t(n_qgroups);
            int qg = int(cluster_id % uint32_t(n_qgroups));
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
                for (int s = 0; s < n_slabs && ok; ++s, ++it) {
                    const int st = it % kStages;
                    ok = mbar_wait(&sh->empty[st], ((it / kStages) & 1) ^ 1, p.cb.error);
                    if (!ok) break;
                    const uint32_t leader_full = map_to_cta(smem_u32(&sh->full[st]), 0);
                    unsigned char *a_tile = stages + size_t(st) * kStageBytes;
                    if (p.live_blocks == nullptr) {
                        mbar_arrive_expect_tx_cluster(leader_full, uint32_t(kStageBytes));
                        tma_load_2d_pair(a_tile, &amap128, s * kSlabK, row0, leader_full);
                    } else {
                        mbar_arrive_expect_tx_cluster(leader_full, uint32_t(n_rows) * 32u * kSlabK + kBHalfBytes);
#pragma unroll
                        for (int b = 0; b < kBlocksPerCta; ++b)
                            if (b < n_rows) tma_load_2d_pair(a_tile + b * 32 * kSlabK, &amap, s * kSlabK, rows[b], leader_full);
                    }
                    tma_load_2d_pair(a_tile + kATileBytes, &wmap, s * kSlabK, qg * kTileQueries + int(rank) * 128, leader_full);
                }
                vt += vt_step; qg += qg_step;
                if (qg >= n_qgroups) { qg -= n_qgroups; ++vt; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer: the leader, for both CTAs -----------------
        if (lane == 0 && rank == 0) {
            uint32_t it = 0, local_item = 0;
            bool ok = true;
            for (uint32_t item = cluster_id; item < n_items && ok; item += n_clusters, ++local_item) {
                const int buf = local_item & 1;
                ok = mbar_wait(&sh->d_empty[buf], ((local_item >> 1) & 1) ^ 1, p.cb.error);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + uint32_t(buf) * kTileQueries;
                for (int s = 0; s < n_slabs && ok; ++s, ++it) {
                    const int st = it % kStages;
                    ok = mbar_wait(&sh->full[st], (it / kStages) & 1, p.cb.error);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(stages + size_t(st) * kStageBytes);
                    const uint32_t b_addr = a_addr + kATileBytes;
#pragma unroll
                    for (int k = 0; k < kSlabK / 32; ++k)
                        umma_i8_pair(d_tmem, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), (s | k) != 0);
                    // the stage may be refilled in both CTAs once these MMAs have read it
                    const uint32_t e = smem_u32(&sh->empty[st]);
                    umma_commit_pair(e);
                    umma_commit_pair(map_to_cta(e, 1));
                }
                if (ok) {
                    const uint32_t f = smem_u32(&sh->d_full[buf]);
                    umma_commit_pair(f);
                    umma_commit_pair(map_to_cta(f, 1));
                }
            }
        }
    } else if (warp >= kFirstEpilogueWarp) {
        // ------------------------------------------------ epilogue: this CTA's 128 vectors x 256 queries --------
        const int quarter = warp & 3;                     // TMEM lanes 32*quarter .. +31 are this warp's
        const int chalf = (warp - kFirstEpilogueWarp) >> 2;   // which 128 of the item's 256 query columns
        const int et = (warp - kFirstEpilogueWarp) * 32 + lane;   // 0..255 among the epilogue threads
        uint32_t local_item = 0;
        uint32_t vt = cluster_id / uint32_t(n_qgroups);
        int qg = int(cluster_id % uint32_t(n_qgroups));
        bool ok = true;
        for (uint32_t item = cluster_id; item < n_items; item += n_clusters, ++local_item) {
            const int buf = local_item & 1;
            // this lane's vector, and the largest vector scale of this CTA's tile (dismissal_bound)
            const int row = quarter * 32 + lane;
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
                if (lane == 0) sh->vs_part[chalf][quarter] = m;
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const float vs_max = fmaxf(fmaxf(sh->vs_part[0][0], sh->vs_part[0][1]), fmaxf(sh->vs_part[0][2], sh->vs_part[0][3]));
            {
                const int ql = qg * kTileQueries + et;
                float qs = 0.f, qb = 0.f, th = INFINITY;
                if (ql < p.q_base + p.nq) {
                    qs = p.qscale[ql]; qb = p.qbias[ql];
                    const uint64_t key = p.cb.thr[ql];
                    th = key == kEmptyKey ? -INFINITY : desc_bits_to_score(uint32_t(key >> 32));
                }
                sh->qscale[et] = qs; sh->qbias[et] = qb; sh->qthr[et] = th;
                sh->ibound[et] = dismissal_bound(qs, qb, th, vs_max);
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");

            const int cbase = chalf * 128;                               // first of this warp's columns
            const float *qscale = sh->qscale + cbase, *qbias = sh->qbias + cbase, *qthr = sh->qthr + cbase;
            // warp-uniform outcome; a warp whose wait ran out still meets the others at the barrier below
            ok = __all_sync(kFullMask, mbar_wait(&sh->d_full[buf], (local_item >> 1) & 1, p.cb.error));
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(buf) * kTileQueries + uint32_t(cbase);
            for (int c0 = 0; c0 < (ok ? 128 : 0); c0 += 32) {
                uint32_t acc[32];
                tmem_ld32(taddr + c0, acc);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (p.dense) {
                    // first chunk of a search: every vector's key goes to the list position of its place in the chunk
                    const uint32_t at = ((vt * 2 + rank) * kBlocksPerCta) * 32u + uint32_t(row);
                    if (have_row)
                        write_piece<ONEHOT>(acc, qscale + c0, qbias + c0, fused, vs, live, slot, qg * kTileQueries + cbase + c0, p.q_base + p.nq, at, p.cb);
                    continue;
                }
                sift_piece<ONEHOT>(acc, sh->ibound + cbase + c0, qscale + c0, qbias + c0, qthr + c0, fused, vs, live, slot,
                                   qg * kTileQueries + cbase + c0, taddr + c0, p.cb);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&sh->d_empty[buf]), 0));   // the leader's barrier counts both CTAs
            // the parameters are rewritten for the next item only after every warp is done with them; the barriers of
            // the next item need all eight warps, so one warp's failure ends the loop of all
            if (!ok && lane == 0) sh->epilogue_failed = 1;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (sh->epilogue_failed) break;
            vt += vt_step; qg += qg_step;
            if (qg >= n_qgroups) { qg -= n_qgroups; ++vt; }
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
    const size_t smem = size_t(kStages) * kStageBytes + sizeof(DensePairShared) + 1024;
    const uint32_t vtiles = (p.pos_end - p.pos_begin + 2 * kBlocksPerCta - 1) / (2 * kBlocksPerCta);
    const uint64_t items = uint64_t(vtiles) * n_qgroups;
    // clusters of two CTAs; a multiple of the query-group count keeps the clusters that share a vector tile in step
    unsigned clusters = unsigned(sm_count / 2);
    clusters -= clusters % unsigned(n_qgroups);
    if (clusters == 0) clusters = unsigned(sm_count / 2);
    if (items < clusters) clusters = unsigned(items);
    cudaError_t e = cudaFuncSetAttribute(scan_tc_dense_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
    scan_tc_dense_pair_kernel<<<clusters * 2, kPairThreads, smem, s>>>(p, amap, amap128, wmap, n_slabs, n_qgroups);
    return cudaGetLastError();
}

}  // namespace tv
