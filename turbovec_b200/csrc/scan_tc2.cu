// Permute-dot scan on CTA pairs: tcgen05.mma.cta_group::2 (M = 256 across two SMs), accumulators in the tensor
// memory of both.
//
// Same arithmetic and the same warp roles as scan_tc_kernel (scan_tc.cu).  What changes is who holds the operands.
// A work item is 256 vectors x 256 queries, run by a cluster of two CTAs on neighbouring SMs:
//   * each CTA expands the codes of ITS 128 vectors into its own A slab (128 rows x 128 B per stage);
//   * each CTA loads ONE HALF of the query slab (128 queries x 128 B per stage) by TMA into its own shared memory;
//     the MMA of the pair reads both halves, so every SM pulls half the query bytes through L2 per multiply-add
//     that the one-CTA kernel does (its query stream, 32 KB per 4 MMAs per SM, is what capped it);
//   * the even CTA of the pair (the leader) issues the MMAs for both; each CTA's 128 x 256 accumulator tile lands
//     in its own tensor memory and is drained by its own epilogue warps.
// Barriers: `full` and `d_empty` live in the leader and collect arrivals from both CTAs (remote mbarrier arrives,
// TMA transactions addressed to the leader's barrier); `empty` and `d_full` exist in both CTAs and the leader
// commits to each.  No load is multicast.
//
// Every wait is bounded; a role whose wait runs out records the error and leaves its loop, and both CTAs always
// meet at the closing cluster barrier.
#include <cuda.h>

#include <algorithm>
#include <cstddef>

#include "scan_tc_common.cuh"

namespace tv {
namespace {

constexpr int kPairStages = 6;                                // 6 x (16 KB A + 16 KB B half) = 192 KB
constexpr int kPairBBytes = 128 * kSlabK;                     // this CTA's half of the query slab
constexpr int kPairStageBytes = kATileBytes + kPairBBytes;
constexpr int kPairItemBlocks = 8;                            // code blocks per work item (4 per CTA)

struct PairShared {
    uint64_t full[kPairStages];    // leader's copy counts: 16 expansion warps + 2 producers (with their TMA bytes)
    uint64_t empty[kPairStages];   // per CTA: stage drained by the pair's MMAs
    uint64_t d_full[2];            // per CTA: accumulator buffer complete
    uint64_t d_empty[2];           // leader's copy counts: 16 epilogue warps
    uint32_t tmem_base;
    uint32_t pad[3];
    float qscale[2][kMaxTileQueries];
    float qbias[2][kMaxTileQueries];
    float qthr[2][kMaxTileQueries];
};
static_assert(offsetof(PairShared, qscale) % 16 == 0, "parameter arrays must be 16-byte aligned");

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreadsTc, 1)
scan_tc_pair_kernel(ScanParams p, const __grid_constant__ CUtensorMap wmap, int n_slabs, int n_qgroups) {
    constexpr int kTileQueries = kMaxTileQueries;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *stages = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    PairShared *sh = reinterpret_cast<PairShared *>(stages + size_t(kPairStages) * kPairStageBytes);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_ctarank();                  // 0 = leader
    const uint32_t cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const int ng = p.ngroups;
    uint32_t pos_end = p.pos_end;
    if (p.live_blocks != nullptr) pos_end = min(pos_end, *p.n_live);
    const uint32_t pos_begin = min(p.pos_begin, pos_end);
    const uint32_t n_vpairs = (pos_end - pos_begin + kPairItemBlocks - 1) / kPairItemBlocks;
    const uint32_t n_items = n_vpairs * uint32_t(n_qgroups);

    if (tid == 0) {
        for (int s = 0; s < kPairStages; ++s) { mbar_init(&sh->full[s], 2 * kExpandWarps + 2); mbar_init(&sh->empty[s], 1); }
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
    // item -> (vector pair, query group), advanced without divisions
    const uint32_t vp_step = n_clusters / uint32_t(n_qgroups);
    const int qg_step = int(n_clusters % uint32_t(n_qgroups));

    if (warp == 0) {
        // ------------------------------------------------ TMA producer: this CTA's half of the query slab ----
        if (lane == 0) {
            uint32_t it = 0;
            int qg = int(cluster_id % uint32_t(n_qgroups));
            bool ok = true;
            for (uint32_t item = cluster_id; item < n_items && ok; item += n_clusters) {
                for (int s = 0; s < n_slabs && ok; ++s, ++it) {
                    const int st = it % kPairStages;
                    ok = mbar_wait_cluster(&sh->empty[st], ((it / kPairStages) & 1) ^ 1, p.cb.error);
                    if (!ok) break;
                    const uint32_t leader_full = map_to_cta(smem_u32(&sh->full[st]), 0);
                    mbar_arrive_expect_tx_cluster(leader_full, kPairBBytes);
                    tma_load_2d_pair(stages + size_t(st) * kPairStageBytes + kATileBytes, &wmap, s * kSlabK,
                                     qg * kTileQueries + int(rank) * 128, leader_full);
                }
                qg += qg_step;
                if (qg >= n_qgroups) qg -= n_qgroups;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer: the leader, for both CTAs -----------------
        if (lane == 0 && rank == 0) {
            uint32_t it = 0, local_item = 0;
            bool ok = true;
            for (uint32_t item = cluster_id; item < n_items && ok; item += n_clusters, ++local_item) {
                const int buf = local_item & 1;
                ok = mbar_wait_cluster(&sh->d_empty[buf], ((local_item >> 1) & 1) ^ 1, p.cb.error);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + uint32_t(buf) * kTileQueries;
                for (int s = 0; s < n_slabs && ok; ++s, ++it) {
                    const int st = it % kPairStages;
                    ok = mbar_wait_cluster(&sh->full[st], (it / kPairStages) & 1, p.cb.error);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(stages + size_t(st) * kPairStageBytes);
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
    } else if (warp < 2 + kEpilogueWarps) {
        // ------------------------------------------------ epilogue: this CTA's 128 vectors x 256 queries --------
        const int quarter = warp & 3;                     // TMEM lanes 32*quarter .. +31 are this warp's
        const int half = (warp - 2) >> 2;                 // which 128 of the item's 256 query columns
        const int et = (warp - 2) * 32 + lane;            // 0..255 among the epilogue threads
        uint32_t local_item = 0;
        uint32_t vp = cluster_id / uint32_t(n_qgroups);
        int qg = int(cluster_id % uint32_t(n_qgroups));
        bool ok = true;
        for (uint32_t item = cluster_id; item < n_items && ok; item += n_clusters, ++local_item) {
            const int buf = local_item & 1, pb = local_item & 1;
            {
                const int ql = qg * kTileQueries + et;
                float qs = 0.f, qb = 0.f, th = INFINITY;
                if (ql < p.q_base + p.nq) {
                    qs = p.qscale[ql]; qb = p.qbias[ql];
                    const uint64_t key = p.cb.thr[ql];
                    th = key == kEmptyKey ? -INFINITY : desc_bits_to_score(uint32_t(key >> 32));
                }
                sh->qscale[pb][et] = qs; sh->qbias[pb][et] = qb; sh->qthr[pb][et] = th;
            }
            asm volatile("bar.sync 1, %0;" ::"r"(kEpilogueWarps * 32) : "memory");
            const int row = quarter * 32 + lane;                         // vector within this CTA's tile
            const uint32_t pos = pos_begin + vp * kPairItemBlocks + rank * 4 + uint32_t(row >> 5);
            const bool have_row = pos < pos_end;
            uint32_t blk = 0;
            if (have_row) blk = p.live_blocks ? p.live_blocks[pos] : pos;
            const int64_t slot = int64_t(blk) * 32 + (row & 31);
            bool live = have_row && slot < p.n;
            if (live && p.mask) live = (p.mask[slot >> 6] >> (slot & 63)) & 1ull;
            const float vs = live ? p.vec_scales[slot] : 0.0f;

            ok = mbar_wait_cluster(&sh->d_full[buf], (local_item >> 1) & 1, p.cb.error);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            constexpr int kColsPerHalf = kTileQueries / 2;
            const int cbase = half * kColsPerHalf;
            const float4 *ps = reinterpret_cast<const float4 *>(&sh->qscale[pb][cbase]);
            const float4 *pbias = reinterpret_cast<const float4 *>(&sh->qbias[pb][cbase]);
            const float4 *pt = reinterpret_cast<const float4 *>(&sh->qthr[pb][cbase]);
            const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(buf) * kTileQueries + uint32_t(cbase);
            for (int c0 = 0; c0 < kColsPerHalf; c0 += 32) {
                uint32_t acc[32];
                tmem_ld32(taddr + c0, acc);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (p.dense) {
                    // first chunk of a search: every vector's key goes to the list position of its place in the chunk
                    const uint32_t at = (vp * kPairItemBlocks + rank * 4) * 32u + uint32_t(row);
                    if (have_row) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int c = cbase + c0 + j;
                            const int ql = qg * kTileQueries + c;
                            if (ql < p.q_base + p.nq) {
                                const float score = final_score<false>(false, acc[j], sh->qscale[pb][c], sh->qbias[pb][c], vs);
                                p.cb.cand[size_t(ql) * p.cb.cap + at] = live ? make_key(score, uint32_t(slot)) : kEmptyKey;
                            }
                        }
                    }
                    continue;
                }
                bool any = false;
#pragma unroll
                for (int j4 = 0; j4 < 8; ++j4) {
                    const float4 s4 = ps[(c0 >> 2) + j4], b4 = pbias[(c0 >> 2) + j4], t4 = pt[(c0 >> 2) + j4];
                    any |= final_score<false>(false, acc[4 * j4 + 0], s4.x, b4.x, vs) >= t4.x;
                    any |= final_score<false>(false, acc[4 * j4 + 1], s4.y, b4.y, vs) >= t4.y;
                    any |= final_score<false>(false, acc[4 * j4 + 2], s4.z, b4.z, vs) >= t4.z;
                    any |= final_score<false>(false, acc[4 * j4 + 3], s4.w, b4.w, vs) >= t4.w;
                }
                any = any && live;
                if (__any_sync(kFullMask, any)) {              // rare, warp-uniform: re-read in pieces of 8 and append
#pragma unroll 1
                    for (int c1 = 0; c1 < 32; c1 += 8) {
                        uint32_t a8[8];
                        tmem_ld8(taddr + c0 + c1, a8);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (any) {
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                const int c = cbase + c0 + c1 + e;
                                const float score = final_score<false>(false, a8[e], sh->qscale[pb][c], sh->qbias[pb][c], vs);
                                if (score >= sh->qthr[pb][c]) {
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
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&sh->d_empty[buf]), 0));
            vp += vp_step; qg += qg_step;
            if (qg >= n_qgroups) { qg -= n_qgroups; ++vp; }
        }
    } else {
        // ------------------------------------------------ expansion: this CTA's codes -> its int8 A slabs --------
        constexpr int kAhead = 4;
        const int ew = warp - (2 + kEpilogueWarps);       // 0..7
        const int octet = lane & 7;                       // which 8-group run of the slab = 16-byte chunk index
        const int blk_in_tile = ew >> 1;
        const int quad0 = (ew & 1) * 4 + (lane >> 3);
        const uint32_t T[4] = {p.level_words[0], p.level_words[1], p.level_words[2], p.level_words[3]};
        const uint32_t my_items = cluster_id < n_items ? (n_items - cluster_id + n_clusters - 1) / n_clusters : 0;
        const uint32_t total = my_items * uint32_t(n_slabs);
        uint32_t w[kAhead][8];
        uint32_t f_item = cluster_id, f_vp = cluster_id / uint32_t(n_qgroups);
        int f_qg = int(cluster_id % uint32_t(n_qgroups)), f_slab = 0;
        const uint32_t *f_src = nullptr;
        bool f_have = false;
        auto fetch = [&](uint32_t (&dst)[8]) {
            if (f_slab == 0) {                            // first slab of an item: locate its code block
                const uint32_t pos = pos_begin + f_vp * kPairItemBlocks + rank * 4 + uint32_t(blk_in_tile);
                f_have = f_item < n_items && pos < pos_end;
                uint32_t blk = 0;
                if (f_have) blk = p.live_blocks ? p.live_blocks[pos] : pos;
                f_src = reinterpret_cast<const uint32_t *>(p.codes + size_t(blk) * ng * 32) + quad0;
            }
            const int g0 = f_slab * (kSlabK / 2) + octet * 8;
            const uint32_t *src = f_src + size_t(g0) * 8;
            const bool whole = f_have && g0 + 8 <= ng;
#pragma unroll
            for (int r = 0; r < 8; ++r) dst[r] = (whole || (f_have && g0 + r < ng)) ? __ldg(src + r * 8) : 0u;
            if (++f_slab == n_slabs) {
                f_slab = 0;
                f_item += n_clusters; f_vp += vp_step; f_qg += qg_step;
                if (f_qg >= n_qgroups) { f_qg -= n_qgroups; ++f_vp; }
            }
        };
#pragma unroll
        for (int a = 0; a < kAhead; ++a) fetch(w[a]);
        bool ok = true;
        for (uint32_t f0 = 0; f0 < total && ok; f0 += kAhead) {
#pragma unroll
            for (int a = 0; a < kAhead; ++a) {
                const uint32_t f = f0 + uint32_t(a);
                if (f >= total || !ok) break;
                const int st = f % kPairStages;
                uint4 v[4];
                {
                    // 4x4 byte transposes: bytes of vector j of the unit in groups g0..g0+3 (xlo) and g0+4..g0+7 (xhi)
                    const uint32_t *x = w[a];
                    const uint32_t t0 = prmt(x[0], x[1], 0x5140), t1 = prmt(x[0], x[1], 0x7362);
                    const uint32_t t2 = prmt(x[2], x[3], 0x5140), t3 = prmt(x[2], x[3], 0x7362);
                    const uint32_t u0 = prmt(x[4], x[5], 0x5140), u1 = prmt(x[4], x[5], 0x7362);
                    const uint32_t u2 = prmt(x[6], x[7], 0x5140), u3 = prmt(x[6], x[7], 0x7362);
                    const uint32_t xlo[4] = {prmt(t0, t2, 0x5410), prmt(t0, t2, 0x7632), prmt(t1, t3, 0x5410), prmt(t1, t3, 0x7632)};
                    const uint32_t xhi[4] = {prmt(u0, u2, 0x5410), prmt(u0, u2, 0x7632), prmt(u1, u3, 0x5410), prmt(u1, u3, 0x7632)};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        expand8(xlo[j], T, v[j].x, v[j].y);
                        expand8(xhi[j], T, v[j].z, v[j].w);
                    }
                }
                fetch(w[a]);                              // refill this ring slot (slab f + kAhead)
                ok = mbar_wait_cluster(&sh->empty[st], ((f / kPairStages) & 1) ^ 1, p.cb.error);
                if (!ok) break;
                unsigned char *a_stage = stages + size_t(st) * kPairStageBytes;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = blk_in_tile * 32 + quad0 * 4 + j;      // vector within this CTA's tile
                    // 128-byte swizzle: 16-byte chunk c of row r sits at chunk position c ^ (r % 8)
                    *reinterpret_cast<uint4 *>(a_stage + (r >> 3) * 1024 + (r & 7) * 128 + ((octet ^ (r & 7)) << 4)) = v[j];
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the MMA
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&sh->full[st]), 0));
            }
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

bool scan_tc_pair_supported(int bits, int mode, int nq_total) {
    return mode == kModePermuteDot && bits == 4 && nq_total > 64 && tensor_map_encoder() != nullptr;
}

// Permute-dot only; weights as for launch_scan_tc (rows a multiple of 256, pitch a multiple of 128).
cudaError_t launch_scan_tc_pair(const ScanParams &p, const int8_t *weights, int rows, int pitch, int sm_count, cudaStream_t s) {
    if (p.nq <= 0 || p.pos_end <= p.pos_begin) return cudaSuccess;
    typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                      const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(tensor_map_encoder());
    if (!enc) return cudaErrorNotSupported;
    const int nq_all = p.q_base + p.nq;
    CUtensorMap map;
    const cuuint64_t dims[2] = {cuuint64_t(pitch), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(pitch)};
    const cuuint32_t box[2] = {cuuint32_t(kSlabK), 128u};     // one CTA's half of a query slab
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t *>(weights), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    const int n_slabs = pitch / kSlabK;
    const int n_qgroups = (nq_all + kMaxTileQueries - 1) / kMaxTileQueries;
    const size_t smem = size_t(kPairStages) * kPairStageBytes + sizeof(PairShared) + 1024;
    cudaError_t e = cudaFuncSetAttribute(scan_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
    const uint32_t vpairs = (p.pos_end - p.pos_begin + kPairItemBlocks - 1) / kPairItemBlocks;
    const uint64_t items = uint64_t(vpairs) * n_qgroups;
    // clusters of two CTAs; a multiple of the query-group count keeps the clusters that share a vector pair in step
    unsigned clusters = unsigned(sm_count / 2);
    clusters -= clusters % unsigned(n_qgroups);
    if (clusters == 0) clusters = unsigned(sm_count / 2);
    if (items < clusters) clusters = unsigned(items);
    scan_tc_pair_kernel<<<clusters * 2, kThreadsTc, smem, s>>>(p, map, n_slabs, n_qgroups);
    return cudaGetLastError();
}

}  // namespace tv
