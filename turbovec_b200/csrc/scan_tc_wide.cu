// Tensor-memory scan for batches of more than 256 queries: every expanded code slab serves TWO query groups.
//
// Same arithmetic, MMA shape and warp roles as scan_tc_kernel (scan_tc.cu): M = 128 vectors x N = 256 queries x
// K = 32, tcgen05.mma kind::i8, accumulators in tensor memory, 8 expansion warps turning 4-bit codes (or, for the
// u8-LUT family, nibbles into one-hots) into the A operand, the B operand (int8 query weights / u8 tables) by TMA.
// In that kernel a work item is 128 vectors x ONE group of 256 queries, so with 1,024 queries every code tile is
// fetched and expanded four times, and the expansion - byte permutes on two warps per scheduler - is what the MMA
// issuer waits for.  Here a work item is 128 vectors x TWO query groups:
//   * the A slabs (128 vectors x 128 bytes of K) go through their own ring of 3 slots; each is expanded once and read
//     by the MMAs of both groups before it is released;
//   * the B slabs (256 queries x 128 bytes, one per group and K slab) go through a ring of 5 slots of their own;
//   * group j of an item accumulates in tensor-memory columns 256 j .. 256 j + 255; the four epilogue warps of half j
//     drain it and hand it back on their own barrier, so the first MMAs of the next item's group 0 wait only for
//     half 0 and overlap the drain of half 1.
// The MMAs of an item's two groups are issued by two threads (warps 1 and 18), one per group.
// An odd last group runs as an item of one group.  Every wait is bounded; a role whose wait runs out records the
// error and leaves its loop.
#include <cuda.h>

#include <algorithm>
#include <cstddef>

#include "scan_tc_common.cuh"

namespace tv {
namespace {

constexpr int kWideASlots = 3;
constexpr int kWideBSlots = 5;
constexpr int kWideBBytes = kMaxTileQueries * kSlabK;        // 32 KB: one query group, one K slab
constexpr int kWideBlocksPerItem = 4;
constexpr int kWideIssuerWarp = 2 + kEpilogueWarps + kExpandWarps;   // warp 18: the MMA issuer of an item's second group
constexpr int kWideThreads = kThreadsTc + 32;

struct WideShared {
    uint64_t a_full[kWideASlots];     // slab expanded: 8 expansion warps
    uint64_t a_empty[kWideASlots];    // slab read by the MMAs of every group of the item (tcgen05.commit)
    uint64_t b_full[kWideBSlots];     // TMA transaction complete
    uint64_t b_empty[kWideBSlots];    // slab read by its 4 MMAs
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
static_assert(offsetof(WideShared, qscale) % 16 == 0, "parameter arrays must be 16-byte aligned");

template <bool ONEHOT>
__global__ void __launch_bounds__(kWideThreads, 1)
scan_tc_wide_kernel(ScanParams p, const __grid_constant__ CUtensorMap wmap, int n_slabs, int n_qgroups) {
    constexpr int kTileQueries = kMaxTileQueries;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *a_ring = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char *b_ring = a_ring + size_t(kWideASlots) * kATileBytes;
    WideShared *sh = reinterpret_cast<WideShared *>(b_ring + size_t(kWideBSlots) * kWideBBytes);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ng = p.ngroups;
    const bool fused = p.mode == kModeLutFlush;          // u8-LUT flush family: one fma per (at most 256) byte-groups
    uint32_t pos_end = p.pos_end;
    if (p.live_blocks != nullptr) pos_end = min(pos_end, *p.n_live);
    const uint32_t pos_begin = min(p.pos_begin, pos_end);
    const uint32_t n_vtiles = (pos_end - pos_begin + kWideBlocksPerItem - 1) / kWideBlocksPerItem;
    const int n_gpairs = (n_qgroups + 1) / 2;
    const uint32_t n_items = n_vtiles * uint32_t(n_gpairs);

    if (tid == 0) {
        for (int s = 0; s < kWideASlots; ++s) { mbar_init(&sh->a_full[s], kExpandWarps); mbar_init(&sh->a_empty[s], 2); }
        for (int s = 0; s < kWideBSlots; ++s) { mbar_init(&sh->b_full[s], 1); mbar_init(&sh->b_empty[s], 1); }
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
        // ------------------------------------------------ TMA producer: query slabs, group by group ------------
        if (lane == 0) {
            uint32_t it = 0;
            int gp = int(blockIdx.x % uint32_t(n_gpairs));
            bool ok = true;
            for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                const int gcount = groups_of(gp);
                for (int s = 0; s < n_slabs && ok; ++s) {
                    for (int j = 0; j < gcount && ok; ++j, ++it) {
                        const int slot = it % kWideBSlots;
                        ok = mbar_wait(&sh->b_empty[slot], ((it / kWideBSlots) & 1) ^ 1, p.cb.error);
                        if (!ok) break;
                        mbar_arrive_expect_tx(&sh->b_full[slot], kWideBBytes);
                        tma_load_2d(b_ring + size_t(slot) * kWideBBytes, &wmap, s * kSlabK, (2 * gp + j) * kTileQueries, &sh->b_full[slot]);
                    }
                }
                gp += gp_step;
                if (gp >= n_gpairs) gp -= n_gpairs;
            }
        }
    } else if (warp == 1 || warp == kWideIssuerWarp) {
        // ------------------------------------------------ MMA issuers: warp 1 for group 0, warp 18 for group 1 --------
        // One thread per group: waiting on a barrier and issuing four MMAs each take a few hundred cycles of the
        // issuing thread, about what the four MMAs take to run, so a single issuer leaves the tensor pipe idle while it
        // waits.  The two groups write different tensor-memory columns, so their MMAs need no order between them.
        if (lane == 0) {
            const int j = warp == 1 ? 0 : 1;                  // this issuer's group within every item
            uint32_t it_a = 0, b_base = 0, uses = 0;
            int gp = int(blockIdx.x % uint32_t(n_gpairs));
            bool ok = true;
            for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                const int gcount = groups_of(gp);
                if (j < gcount) {
                    for (int s = 0; s < n_slabs && ok; ++s) {
                        const uint32_t ia = it_a + uint32_t(s);
                        const int a_slot = ia % kWideASlots;
                        if (s == 0) {                         // the half must have been drained by the previous item's epilogue
                            ok = mbar_wait(&sh->d_empty[j], (uses & 1) ^ 1, p.cb.error);
                            if (!ok) break;
                        }
                        ok = mbar_wait(&sh->a_full[a_slot], (ia / kWideASlots) & 1, p.cb.error);
                        if (!ok) break;
                        const uint32_t ib = b_base + uint32_t(s * gcount + j);
                        const int b_slot = ib % kWideBSlots;
                        ok = mbar_wait(&sh->b_full[b_slot], (ib / kWideBSlots) & 1, p.cb.error);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t a_addr = smem_u32(a_ring + size_t(a_slot) * kATileBytes);
                        const uint32_t b_addr = smem_u32(b_ring + size_t(b_slot) * kWideBBytes);
                        const uint32_t d_tmem = tmem_base + uint32_t(j) * kTileQueries;
#pragma unroll
                        for (int k = 0; k < kSlabK / 32; ++k)
                            umma_i8<kTileQueries>(d_tmem, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), (s | k) != 0);
                        umma_commit(&sh->b_empty[b_slot]);
                        umma_commit(&sh->a_empty[a_slot]);    // the slab is free once both groups have read it
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
    } else if (warp < 2 + kEpilogueWarps) {
        // ------------------------------------------------ epilogue: warps of half j drain group j of the item ----
        const int quarter = warp & 3;                     // TMEM lanes 32*quarter .. +31 are this warp's
        const int half = (warp - 2) >> 2;                 // which group of the item
        const int ht = ((warp - 2) & 3) * 32 + lane;      // 0..127 among the threads of this half
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
                const uint32_t pos = pos_begin + vt * kWideBlocksPerItem + uint32_t(row >> 5);
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
                        const uint32_t at = (vt * kWideBlocksPerItem) * 32u + uint32_t(row);
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
    } else if (warp < kWideIssuerWarp) {
        // ------------------------------------------------ expansion: codes -> int8 A slabs, once per item and slab ----
        constexpr int kAhead = 4;
        const int ew = warp - (2 + kEpilogueWarps);       // 0..7
        const int octet = lane & 7;                       // which 8-group run of the slab = 16-byte chunk index
        const int blk_in_item = ew >> 1;
        const int quad0 = (ew & 1) * 4 + (lane >> 3);
        const uint32_t T[4] = {p.level_words[0], p.level_words[1], p.level_words[2], p.level_words[3]};
        const uint32_t my_items = blockIdx.x < n_items ? (n_items - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        const uint32_t total = my_items * uint32_t(n_slabs);
        constexpr int kWords = ONEHOT ? 1 : 8;            // code words per thread and slab
        uint32_t w[kAhead][kWords];
        uint32_t f_item = blockIdx.x, f_vt = blockIdx.x / uint32_t(n_gpairs);
        int f_gp = int(blockIdx.x % uint32_t(n_gpairs)), f_slab = 0;
        const uint32_t *f_src = nullptr;
        bool f_have = false;
        auto fetch = [&](uint32_t (&dst)[kWords]) {
            if (f_slab == 0) {                            // first slab of an item: locate its code block
                const uint32_t pos = pos_begin + f_vt * kWideBlocksPerItem + uint32_t(blk_in_item);
                f_have = f_item < n_items && pos < pos_end;
                uint32_t blk = 0;
                if (f_have) blk = p.live_blocks ? p.live_blocks[pos] : pos;
                f_src = reinterpret_cast<const uint32_t *>(p.codes + size_t(blk) * ng * 32) + quad0;
            }
            if constexpr (ONEHOT) {
                // a slab is 4 byte-groups x 32 table entries; chunk `octet` = group octet/2, nibble octet%2
                const int g = f_slab * 4 + (octet >> 1);
                dst[0] = (f_have && g < ng) ? __ldg(f_src + size_t(g) * 8) : 0u;
            } else {
                const int g0 = f_slab * (kSlabK / 2) + octet * 8;
                const uint32_t *src = f_src + size_t(g0) * 8;
                const bool whole = f_have && g0 + 8 <= ng;
#pragma unroll
                for (int r = 0; r < 8; ++r) dst[r] = (whole || (f_have && g0 + r < ng)) ? __ldg(src + r * 8) : 0u;
            }
            if (++f_slab == n_slabs) {
                f_slab = 0;
                f_item += gridDim.x; f_vt += vt_step; f_gp += gp_step;
                if (f_gp >= n_gpairs) { f_gp -= n_gpairs; ++f_vt; }
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
                const int slot = f % kWideASlots;
                uint4 v[4];
                if constexpr (ONEHOT) {
                    // byte j of the word = code byte of vector j in this chunk's group; its high (even chunk)
                    // or low (odd chunk) nibble n becomes a 16-byte one-hot: byte n = 1
                    const uint32_t word = w[a][0];
                    const uint32_t nibs = (octet & 1) ? (word & 0x0f0f0f0fu) : ((word >> 4) & 0x0f0f0f0fu);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t n = (nibs >> (8 * j)) & 15u;
                        const uint32_t bit = 1u << ((n & 3u) * 8u);
                        const uint32_t q = n >> 2;
                        v[j].x = q == 0 ? bit : 0u; v[j].y = q == 1 ? bit : 0u;
                        v[j].z = q == 2 ? bit : 0u; v[j].w = q == 3 ? bit : 0u;
                    }
                } else {
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
                fetch(w[a]);                              // refill this register slot (slab f + kAhead)
                ok = mbar_wait(&sh->a_empty[slot], ((f / kWideASlots) & 1) ^ 1, p.cb.error);
                if (!ok) break;
                unsigned char *a_slab = a_ring + size_t(slot) * kATileBytes;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = blk_in_item * 32 + quad0 * 4 + j;      // vector within the item
                    // 128-byte swizzle: 16-byte chunk c of row r sits at chunk position c ^ (r % 8)
                    *reinterpret_cast<uint4 *>(a_slab + (r >> 3) * 1024 + (r & 7) * 128 + ((octet ^ (r & 7)) << 4)) = v[j];
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the MMA
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->a_full[slot]);
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

}  // namespace

bool scan_tc_wide_supported(int bits, int mode, int ngroups, int nq_total) {
    return nq_total > kMaxTileQueries && scan_tc_supported(bits, mode, ngroups);
}

// weights / pitch / rows as for launch_scan_tc.
cudaError_t launch_scan_tc_wide(const ScanParams &p, const int8_t *weights, int rows, int pitch, int sm_count, cudaStream_t s) {
    if (p.nq <= 0 || p.pos_end <= p.pos_begin) return cudaSuccess;
    typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                      const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(tensor_map_encoder());
    if (!enc) return cudaErrorNotSupported;
    const bool onehot = p.mode != kModePermuteDot;
    const int nq_all = p.q_base + p.nq;
    CUtensorMap map;
    const cuuint64_t dims[2] = {cuuint64_t(pitch), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(pitch)};
    const cuuint32_t box[2] = {cuuint32_t(kSlabK), cuuint32_t(kMaxTileQueries)};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t *>(weights), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    const int n_slabs = pitch / kSlabK;
    const int n_qgroups = (nq_all + kMaxTileQueries - 1) / kMaxTileQueries;
    const int n_gpairs = (n_qgroups + 1) / 2;
    const size_t smem = size_t(kWideASlots) * kATileBytes + size_t(kWideBSlots) * kWideBBytes + sizeof(WideShared) + 1024;
    const uint32_t vtiles = (p.pos_end - p.pos_begin + kWideBlocksPerItem - 1) / kWideBlocksPerItem;
    const uint64_t items = uint64_t(vtiles) * n_gpairs;
    // a multiple of the group-pair count keeps the CTAs that share a vector tile in step (codes hit L2)
    unsigned grid = unsigned(sm_count - sm_count % n_gpairs);
    if (grid == 0) grid = unsigned(sm_count);
    if (items < grid) grid = unsigned(items);
    cudaError_t e;
    if (onehot) {
        e = cudaFuncSetAttribute(scan_tc_wide_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        scan_tc_wide_kernel<true><<<grid, kWideThreads, smem, s>>>(p, map, n_slabs, n_qgroups);
    } else {
        e = cudaFuncSetAttribute(scan_tc_wide_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        scan_tc_wide_kernel<false><<<grid, kWideThreads, smem, s>>>(p, map, n_slabs, n_qgroups);
    }
    return cudaGetLastError();
}

}  // namespace tv
