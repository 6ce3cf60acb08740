// Permute-dot scan on the 5th-generation tensor cores (tcgen05.mma kind::i8, accumulators in TMEM).
//
// Same arithmetic as scan_pd_kernel (search.cu): S[q][v] = sum_d W[q][d] * level[code[v][d]] exactly in
// int32 (turbovec/src/search.rs:1392-1543), then fma((f32)S, scale_q, bias_q) * vec_scale[v]
// (search.rs:1523, 1793) and the candidate push against the query's current k-th key.
//
// One work item = 128 vectors (4 code blocks) x 256 queries.  MMA shape M = 128 (vectors) x N = 256
// (queries) x K = 32, both operands K-major in shared memory with the 128-byte swizzle:
//   A (vectors): 4-bit codes are read from global memory and expanded to int8 levels by 8 CUDA-core warps,
//      one 128-dimension slab (128 rows x 128 B) per pipeline stage;
//   B (queries): int8 weights, one 256 x 128 B box per stage, loaded by TMA (no multicast).
// D (128 lanes x 256 int32 columns) lives in TMEM, double buffered (512 columns), so the epilogue of one
// work item overlaps the MMAs of the next.  Warp roles: 0 = TMA producer, 1 = MMA issuer (+ TMEM
// alloc/dealloc), 2-9 = epilogue (two per TMEM lane quarter, half the columns each), 10-17 = code expansion.
//
// Every wait is bounded; a wait that runs out records an error word and makes its role leave its loop.
#include <cuda.h>

#include <algorithm>

#include <cstddef>

#include "scan_tc_common.cuh"

namespace tv {
namespace {

struct TcShared {
    uint64_t full[4];              // stage filled: 8 expansion warps + the TMA transaction
    uint64_t empty[4];             // stage drained by the MMAs (tcgen05.commit)
    uint64_t d_full[2];            // accumulator buffer complete
    uint64_t d_empty[2];           // accumulator buffer read out by the epilogue warps
    uint32_t tmem_base;
    uint32_t pad[3];
    // per-query parameters of an item, double buffered; 16-byte aligned for float4 loads
    float qscale[2][kMaxTileQueries];
    float qbias[2][kMaxTileQueries];
    float qthr[2][kMaxTileQueries];   // score of the current k-th key (-inf while fewer than k results exist)
    int ibound[2][kMaxTileQueries];   // per query: integer sum below which no vector of the item can be a candidate
    float vs_part[2][8];              // largest vector scale seen by each epilogue warp of the item
};
static_assert(offsetof(TcShared, qscale) % 16 == 0, "parameter arrays must be 16-byte aligned");

// ONEHOT = false: permute-dot.  A rows hold the int8 levels of the codes, B rows the int8 query weights
// (K = dim).  ONEHOT = true: the u8-LUT scan as a contraction (K = 32 * ngroups): A rows hold, per
// byte-group, a one-hot of the high nibble (16 bytes) then a one-hot of the low nibble (16 bytes); B rows are
// the per-query u8 tables exactly as query preparation lays them out ([g][hi 16 | lo 16], entries <= 127),
// so the int32 accumulator is the reference's integer LUT sum (search.rs:1071-1195) and the epilogue applies
// (f32)isum * scale + bias (search.rs:1176).
// MT = accumulator tiles (of 128 vectors) that share one B slab.  MT = 1: work item 128 x 256, four stages,
// two accumulator buffers (the epilogue of an item overlaps the MMAs of the next).  MT = 2: work item
// 256 x 256, three stages, both 256-column halves of TMEM hold one item — half the B traffic per
// multiply-add, at the price of the MMA pipe idling while the epilogue drains the accumulators.
// NQT = query columns of a work item (MMA N): 256, or 64 / 32 for small batches, where a full-width item
// would spend three quarters or more of its tensor time on columns that hold no query.
template <int MT, bool ONEHOT, int NQT>
__global__ void __launch_bounds__(kThreadsTc, 1)
scan_tc_kernel(ScanParams p, const __grid_constant__ CUtensorMap wmap, int n_slabs, int n_qgroups) {
    constexpr int kStages = MT == 1 ? 4 : 3;
    constexpr int kABytes = MT * kATileBytes;
    constexpr int kBBytes = NQT * kSlabK;                     // 32 KB at 256 columns
    constexpr int kStageBytes = kABytes + kBBytes;
    constexpr uint32_t kTmemCols = (MT == 1 ? 2 : 1) * MT * NQT < 32 ? 32 : (MT == 1 ? 2 : 1) * MT * NQT;   // 512 / 128 / 64: powers of two
    constexpr int kTileQueries = NQT;
    constexpr int kBufs = MT == 1 ? 2 : 1;                    // accumulator buffers
    constexpr int kBlocksPerItem = 4 * MT;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // stages first (1024-byte aligned for the swizzle), bookkeeping after them
    unsigned char *stages = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    TcShared *sh = reinterpret_cast<TcShared *>(stages + size_t(kStages) * kStageBytes);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ng = p.ngroups;
    const bool fused = p.mode == kModeLutFlush;          // u8-LUT flush family: one fma per (at most 256) byte-groups
    uint32_t pos_end = p.pos_end;
    if (p.live_blocks != nullptr) pos_end = min(pos_end, *p.n_live);
    const uint32_t pos_begin = min(p.pos_begin, pos_end);
    const uint32_t n_vtiles = (pos_end - pos_begin + kBlocksPerItem - 1) / kBlocksPerItem;
    const uint32_t n_items = n_vtiles * uint32_t(n_qgroups);

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&sh->full[s], kExpandWarps + 1); mbar_init(&sh->empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sh->d_full[b], 1); mbar_init(&sh->d_empty[b], kEpilogueWarps); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = sh->tmem_base;
    // item -> (vector tile, query group), advanced without divisions
    const uint32_t vt_step = gridDim.x / uint32_t(n_qgroups);
    const int qg_step = int(gridDim.x % uint32_t(n_qgroups));

    if (warp == 0) {
        // ------------------------------------------------ TMA producer: query weights ------------
        if (lane == 0) {
            uint32_t it = 0;
            int qg = int(blockIdx.x % uint32_t(n_qgroups));
            bool ok = true;
            for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                for (int s = 0; s < n_slabs && ok; ++s, ++it) {
                    const int st = it % kStages;
                    ok = mbar_wait(&sh->empty[st], ((it / kStages) & 1) ^ 1, p.cb.error);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&sh->full[st], kBBytes);
                    tma_load_2d(stages + size_t(st) * kStageBytes + kABytes, &wmap, s * kSlabK, qg * kTileQueries, &sh->full[st]);
                }
                qg += qg_step;
                if (qg >= n_qgroups) qg -= n_qgroups;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer -----------------------------
        if (lane == 0) {
            uint32_t it = 0, local_item = 0;
            bool ok = true;
            for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++local_item) {
                const int buf = local_item % kBufs;
                ok = mbar_wait(&sh->d_empty[buf], ((local_item / kBufs) & 1) ^ 1, p.cb.error);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + uint32_t(buf * MT) * kTileQueries;
                for (int s = 0; s < n_slabs && ok; ++s, ++it) {
                    const int st = it % kStages;
                    ok = mbar_wait(&sh->full[st], (it / kStages) & 1, p.cb.error);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(stages + size_t(st) * kStageBytes);
                    const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
                    for (int k = 0; k < kSlabK / 32; ++k) {
                        const uint64_t bd = umma_desc(b_addr + k * 32);
#pragma unroll
                        for (int m = 0; m < MT; ++m)
                            umma_i8<NQT>(d_tmem + uint32_t(m) * kTileQueries, umma_desc(a_addr + m * kATileBytes + k * 32), bd, (s | k) != 0);
                    }
                    umma_commit(&sh->empty[st]);          // the stage may be refilled once these MMAs have read it
                }
                if (ok) umma_commit(&sh->d_full[buf]);
            }
        }
    } else if (warp < 2 + kEpilogueWarps) {
        // ------------------------------------------------ epilogue -------------------------------
        const int quarter = warp & 3;                     // TMEM lanes 32*quarter .. +31 are this warp's
        const int half = (warp - 2) >> 2;                 // which 128 of the item's 256 query columns
        const int et = (warp - 2) * 32 + lane;            // 0..255 among the epilogue threads
        uint32_t local_item = 0;
        uint32_t vt = blockIdx.x / uint32_t(n_qgroups);
        int qg = int(blockIdx.x % uint32_t(n_qgroups));
        bool ok = true;
        for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++local_item) {
            const int buf = local_item % kBufs, pb = local_item & 1;
            int64_t slot[MT];
            float vs[MT];
            bool live[MT], have_row[MT];
            float vs_warp = 0.0f;
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const int row = m * kMmaM + quarter * 32 + lane;        // vector within the item
                const uint32_t pos = pos_begin + vt * kBlocksPerItem + uint32_t(row >> 5);
                const bool have = pos < pos_end;
                have_row[m] = have;
                uint32_t blk = 0;
                if (have) blk = p.live_blocks ? p.live_blocks[pos] : pos;
                slot[m] = int64_t(blk) * 32 + (row & 31);
                live[m] = have && slot[m] < p.n;
                if (live[m] && p.mask) live[m] = (p.mask[slot[m] >> 6] >> (slot[m] & 63)) & 1ull;
                vs[m] = live[m] ? p.vec_scales[slot[m]] : 0.0f;
                vs_warp = fmaxf(vs_warp, vs[m]);
            }
            // the largest vector scale of the item, for the integer dismissal bound of every query
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) vs_warp = fmaxf(vs_warp, __shfl_xor_sync(kFullMask, vs_warp, o));
            if (lane == 0) sh->vs_part[pb][warp - 2] = vs_warp;
            asm volatile("bar.sync 1, %0;" ::"r"(kEpilogueWarps * 32) : "memory");
            // per-query parameters of this item: one query per epilogue thread
            {
                float vs_max = 0.0f;
#pragma unroll
                for (int i = 0; i < kEpilogueWarps; ++i) vs_max = fmaxf(vs_max, sh->vs_part[pb][i]);
                const int ql = qg * kTileQueries + et;
                float qs = 0.f, qb = 0.f, th = INFINITY;
                if (et < kTileQueries && ql < p.q_base + p.nq) {
                    qs = p.qscale[ql]; qb = p.qbias[ql];
                    const uint64_t key = p.cb.thr[ql];
                    th = key == kEmptyKey ? -INFINITY : desc_bits_to_score(uint32_t(key >> 32));
                }
                sh->qscale[pb][et] = qs; sh->qbias[pb][et] = qb; sh->qthr[pb][et] = th;
                sh->ibound[pb][et] = dismissal_bound(qs, qb, th, vs_max);
            }
            asm volatile("bar.sync 1, %0;" ::"r"(kEpilogueWarps * 32) : "memory");

            ok = mbar_wait(&sh->d_full[buf], (local_item / kBufs) & 1, p.cb.error);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // the two warps of a lane quarter split the columns; below 64 columns the second one has none
            constexpr int kColsPerHalf = kTileQueries >= 64 ? kTileQueries / 2 : kTileQueries;
            const int cbase = half * kColsPerHalf;
            const bool has_columns = cbase < kTileQueries;
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(buf * MT + m) * kTileQueries + uint32_t(cbase);
                for (int c0 = 0; c0 < (has_columns ? kColsPerHalf : 0); c0 += 32) {
                    uint32_t acc[32];
                    tmem_ld32(taddr + c0, acc);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (p.dense) {
                        // first chunk of a search: every vector's key goes to the list position of its place in the chunk
                        const uint32_t at = (vt * kBlocksPerItem) * 32u + uint32_t(m * kMmaM + quarter * 32 + lane);
                        if (have_row[m])
                            write_piece<ONEHOT>(acc, &sh->qscale[pb][cbase + c0], &sh->qbias[pb][cbase + c0], fused, vs[m], live[m], slot[m],
                                                qg * kTileQueries + cbase + c0, p.q_base + p.nq, at, p.cb);
                        continue;
                    }
                    sift_piece<ONEHOT>(acc, &sh->ibound[pb][cbase + c0], &sh->qscale[pb][cbase + c0], &sh->qbias[pb][cbase + c0], &sh->qthr[pb][cbase + c0],
                                       fused, vs[m], live[m], slot[m], qg * kTileQueries + cbase + c0, taddr + c0, p.cb);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->d_empty[buf]);
            vt += vt_step; qg += qg_step;
            if (qg >= n_qgroups) { qg -= n_qgroups; ++vt; }
        }
    } else {
        // ------------------------------------------------ expansion: codes -> int8 A slabs -------
        // The (item, slab) pairs of this CTA form one flat sequence; the code words of the next kAhead slabs
        // are kept in flight in registers so that global-load latency never reaches the expansion itself.
        // A unit = 4 vectors (one 32-bit column of a code block) x 8 byte-groups (one 16-byte chunk of a row).
        constexpr int kUnits = MT;                        // units per thread and slab
        constexpr int kAhead = MT == 1 ? 4 : 3;
        const int ew = warp - (2 + kEpilogueWarps);       // 0..7
        const int octet = lane & 7;                       // which 8-group run of the slab = 16-byte chunk index
        const int blk_in_item = MT == 1 ? (ew >> 1) : ew;
        const int quad0 = (MT == 1 ? (ew & 1) * 4 : 0) + (lane >> 3);   // unit u handles quad0 + 4u
        const uint32_t T[4] = {p.level_words[0], p.level_words[1], p.level_words[2], p.level_words[3]};
        const uint32_t my_items = blockIdx.x < n_items ? (n_items - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        const uint32_t total = my_items * uint32_t(n_slabs);
        constexpr int kWords = ONEHOT ? 1 : 8;            // code words per unit and slab
        uint32_t w[kAhead][kUnits][kWords];
        // fetch cursor: walks the same (item, slab) sequence as the consumers
        uint32_t f_item = blockIdx.x, f_vt = blockIdx.x / uint32_t(n_qgroups);
        int f_qg = int(blockIdx.x % uint32_t(n_qgroups)), f_slab = 0;
        const uint32_t *f_src = nullptr;
        bool f_have = false;
        auto fetch = [&](uint32_t (&dst)[kUnits][kWords]) {
            if (f_slab == 0) {                            // first slab of an item: locate its code block
                const uint32_t pos = pos_begin + f_vt * kBlocksPerItem + uint32_t(blk_in_item);
                f_have = f_item < n_items && pos < pos_end;
                uint32_t blk = 0;
                if (f_have) blk = p.live_blocks ? p.live_blocks[pos] : pos;
                f_src = reinterpret_cast<const uint32_t *>(p.codes + size_t(blk) * ng * 32) + quad0;
            }
            if constexpr (ONEHOT) {
                // a slab is 4 byte-groups x 32 table entries; chunk `octet` = group octet/2, nibble octet%2
                const int g = f_slab * 4 + (octet >> 1);
#pragma unroll
                for (int u = 0; u < kUnits; ++u) dst[u][0] = (f_have && g < ng) ? __ldg(f_src + size_t(g) * 8 + u * 4) : 0u;
            } else {
                const int g0 = f_slab * (kSlabK / 2) + octet * 8;
                const uint32_t *src = f_src + size_t(g0) * 8;
                const bool whole = f_have && g0 + 8 <= ng;
#pragma unroll
                for (int u = 0; u < kUnits; ++u)
#pragma unroll
                    for (int r = 0; r < 8; ++r)
                        dst[u][r] = (whole || (f_have && g0 + r < ng)) ? __ldg(src + r * 8 + u * 4) : 0u;
            }
            if (++f_slab == n_slabs) {
                f_slab = 0;
                f_item += gridDim.x; f_vt += vt_step; f_qg += qg_step;
                if (f_qg >= n_qgroups) { f_qg -= n_qgroups; ++f_vt; }
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
                const int st = f % kStages;
                uint4 v[kUnits][4];
#pragma unroll
                for (int u = 0; u < kUnits; ++u) {
                    if constexpr (ONEHOT) {
                        // byte j of the word = code byte of vector j in this chunk's group; its high (even chunk)
                        // or low (odd chunk) nibble n becomes a 16-byte one-hot: byte n = 1
                        const uint32_t word = w[a][u][0];
                        const uint32_t nibs = (octet & 1) ? (word & 0x0f0f0f0fu) : ((word >> 4) & 0x0f0f0f0fu);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t n = (nibs >> (8 * j)) & 15u;
                            const uint32_t bit = 1u << ((n & 3u) * 8u);
                            const uint32_t q = n >> 2;
                            v[u][j].x = q == 0 ? bit : 0u; v[u][j].y = q == 1 ? bit : 0u;
                            v[u][j].z = q == 2 ? bit : 0u; v[u][j].w = q == 3 ? bit : 0u;
                        }
                    } else {
                        // 4x4 byte transposes: bytes of vector j of the unit in groups g0..g0+3 (xlo) and g0+4..g0+7 (xhi)
                        const uint32_t *x = w[a][u];
                        const uint32_t t0 = prmt(x[0], x[1], 0x5140), t1 = prmt(x[0], x[1], 0x7362);
                        const uint32_t t2 = prmt(x[2], x[3], 0x5140), t3 = prmt(x[2], x[3], 0x7362);
                        const uint32_t u0 = prmt(x[4], x[5], 0x5140), u1 = prmt(x[4], x[5], 0x7362);
                        const uint32_t u2 = prmt(x[6], x[7], 0x5140), u3 = prmt(x[6], x[7], 0x7362);
                        const uint32_t xlo[4] = {prmt(t0, t2, 0x5410), prmt(t0, t2, 0x7632), prmt(t1, t3, 0x5410), prmt(t1, t3, 0x7632)};
                        const uint32_t xhi[4] = {prmt(u0, u2, 0x5410), prmt(u0, u2, 0x7632), prmt(u1, u3, 0x5410), prmt(u1, u3, 0x7632)};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            expand8(xlo[j], T, v[u][j].x, v[u][j].y);
                            expand8(xhi[j], T, v[u][j].z, v[u][j].w);
                        }
                    }
                }
                fetch(w[a]);                              // refill this ring slot (slab f + kAhead)
                ok = mbar_wait(&sh->empty[st], ((f / kStages) & 1) ^ 1, p.cb.error);
                if (!ok) break;
                unsigned char *a_stage = stages + size_t(st) * kStageBytes;
#pragma unroll
                for (int u = 0; u < kUnits; ++u)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int row = blk_in_item * 32 + (quad0 + 4 * u) * 4 + j;   // vector within the item
                        const int r = row & (kMmaM - 1);
                        // accumulator tile row>>7; 128-byte swizzle: 16-byte chunk c of row r sits at chunk position c ^ (r % 8)
                        *reinterpret_cast<uint4 *>(a_stage + (row >> 7) * kATileBytes + (r >> 3) * 1024 + (r & 7) * 128 + ((octet ^ (r & 7)) << 4)) = v[u][j];
                    }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the MMA
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->full[st]);
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}


// ---- tensor-pipe peak for kind::i8: MMAs issued back to back on shared-memory operands, no loads, no epilogue ----
// One CTA per SM, 1 + 1 warps: warp 0 lane 0 issues M = 128, N = 256, K = 32 MMAs alternating between the two
// accumulator halves of TMEM and commits every 64 of them to one of two barriers, waiting (bounded) for the batch
// before the one just issued, so the issue queue stays two batches deep.  The operands are whatever the shared memory holds: the result is discarded.
__global__ void __launch_bounds__(64, 1) int8_peak_kernel(int batches, uint32_t *error_flag) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *ops = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t done_bar[2];
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < (kATileBytes + kMaxTileQueries * kSlabK) / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(ops)[i] = 0x01010101u;
    if (threadIdx.x == 0) {
        mbar_init(&done_bar[0], 1);
        mbar_init(&done_bar[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    if (warp == 0 && lane == 0) {
        const uint32_t a_addr = smem_u32(ops), b_addr = a_addr + kATileBytes;
        bool ok = true;
        for (int b = 0; b < batches && ok; ++b) {
#pragma unroll 4
            for (int i = 0; i < 64; ++i)
                umma_i8<256>(tmem_base + uint32_t(i & 1) * 256u, umma_desc(a_addr + (i & 3) * 32), umma_desc(b_addr + (i & 3) * 32), 1u);
            umma_commit(&done_bar[b & 1]);
            // wait for the batch before this one: one batch stays queued behind the one that runs
            if (b > 0) ok = mbar_wait(&done_bar[(b - 1) & 1], uint32_t(((b - 1) >> 1) & 1), error_flag);
        }
        if (ok && batches > 0) mbar_wait(&done_bar[(batches - 1) & 1], uint32_t(((batches - 1) >> 1) & 1), error_flag);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

}  // namespace

// Runs int8_peak_kernel on one CTA per SM and returns the int8 rate in ops/s (a multiply-add = 2 ops), 0 on failure.
// seconds <= 0: the best of three launches of about 2 ms (a burst, before the power limit acts); otherwise launches back
// to back for `seconds` and the rate over the second half of that time (what the device sustains at its power limit).
double measure_int8_peak(int sm_count, double seconds, cudaStream_t s) {
    const int batches = 512;                                   // 32,768 MMAs of 2 * 128 * 256 * 32 ops per CTA
    const size_t smem = size_t(kATileBytes) + size_t(kMaxTileQueries) * kSlabK + 1024;
    if (cudaFuncSetAttribute(int8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return 0.0;
    uint32_t *d_err = nullptr;
    if (cudaMalloc(&d_err, 4) != cudaSuccess) return 0.0;
    cudaMemsetAsync(d_err, 0, 4, s);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    int8_peak_kernel<<<sm_count, 64, smem, s>>>(8, d_err);     // warm-up
    const double ops_per_launch = 2.0 * 128 * 256 * 32 * 64.0 * batches * sm_count;
    double best = 0.0;
    if (seconds <= 0.0) {
        for (int rep = 0; rep < 3; ++rep) {
            cudaEventRecord(e0, s);
            int8_peak_kernel<<<sm_count, 64, smem, s>>>(batches, d_err);
            cudaEventRecord(e1, s);
            if (cudaStreamSynchronize(s) != cudaSuccess) { best = 0.0; break; }
            float ms = 0.f;
            cudaEventElapsedTime(&ms, e0, e1);
            if (ms > 0.f) best = std::max(best, ops_per_launch / (double(ms) * 1e-3));
        }
    } else {
        seconds = std::min(seconds, 10.0);
        // a launch takes about 2 ms at full clocks: half the launches warm the device up, the other half are timed
        const int half = std::max(4, int(seconds * 0.5 / 2.2e-3));
        for (int i = 0; i < half; ++i) int8_peak_kernel<<<sm_count, 64, smem, s>>>(batches, d_err);
        cudaEventRecord(e0, s);
        for (int i = 0; i < half; ++i) int8_peak_kernel<<<sm_count, 64, smem, s>>>(batches, d_err);
        cudaEventRecord(e1, s);
        if (cudaStreamSynchronize(s) == cudaSuccess) {
            float ms = 0.f;
            cudaEventElapsedTime(&ms, e0, e1);
            if (ms > 0.f) best = ops_per_launch * half / (double(ms) * 1e-3);
        }
    }
    uint32_t err = 0;
    cudaMemcpy(&err, d_err, 4, cudaMemcpyDeviceToHost);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    cudaFree(d_err);
    cudaGetLastError();
    return err ? 0.0 : best;
}

void *tensor_map_encoder() { return reinterpret_cast<void *>(encode_fn()); }

static size_t scan_tc_smem_bytes(int nqt) { return size_t(4) * (kATileBytes + nqt * kSlabK) + sizeof(TcShared) + 1024; }   // MT = 2: 3 x 64 KB, the same

bool scan_tc_supported(int bits, int mode, int ngroups) {
    if (encode_fn() == nullptr) return false;
    if (mode == kModePermuteDot) return bits == 4;
    if (mode == kModeLutMulAdd) return ngroups % 4 == 0;
    // flush family: acc = bias, then one fma(scale, (f32)isum, acc) per 256 byte-groups (search.rs:516, 577): with at
    // most 256 groups that is a single fma on the whole integer sum, which the accumulator holds; longer rows need the
    // partial sums and stay on the CUDA-core scan.  K is padded to whole slabs of 4 groups with zero tables.
    return mode == kModeLutFlush && ngroups <= 256;
}

// Permute-dot: weights = [rows][pitch] int8, pitch a multiple of 128, rows a multiple of 256, coordinates
// pair-swapped (byte 2g = coordinate 2g+1, byte 2g+1 = coordinate 2g) to match the nibble order of a code byte.
// LUT: weights = the u8 tables [rows][pitch = 32 * ngroups].
// tiles_per_item: 1 or 2 accumulator tiles of 128 vectors per B slab (see the kernel).
cudaError_t launch_scan_tc(const ScanParams &p, const int8_t *weights, int rows, int pitch, int sm_count, int tiles_per_item,
                           cudaStream_t s) {
    if (p.nq <= 0 || p.pos_end <= p.pos_begin) return cudaSuccess;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    const bool onehot = p.mode != kModePermuteDot;
    const int nq_all = p.q_base + p.nq;
    // query columns per work item: the tensor time of an item grows with them whether they hold queries or not
    const int nqt = nq_all <= 32 && onehot ? 32 : (nq_all <= 64 ? 64 : kMaxTileQueries);
    CUtensorMap map;
    const cuuint64_t dims[2] = {cuuint64_t(pitch), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(pitch)};
    const cuuint32_t box[2] = {cuuint32_t(kSlabK), cuuint32_t(nqt)};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t *>(weights), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    const int n_slabs = pitch / kSlabK;
    const int n_qgroups = (nq_all + nqt - 1) / nqt;
    const size_t smem = scan_tc_smem_bytes(nqt);
    const int mt = (tiles_per_item == 2 && !onehot && nqt == kMaxTileQueries) ? 2 : 1;
    const uint32_t vtiles = (p.pos_end - p.pos_begin + 4 * mt - 1) / (4 * mt);
    const uint64_t items = uint64_t(vtiles) * n_qgroups;
    // a multiple of the query-group count keeps the CTAs that share a vector tile in step (codes hit L2)
    unsigned grid = unsigned(sm_count - sm_count % n_qgroups);
    if (grid == 0) grid = unsigned(sm_count);
    if (items < grid) grid = unsigned(items);
    // the shared-memory attribute belongs to the current device: set on every launch (a host-side table write)
#define TV_LAUNCH_TC(M, O, N)                                                                                           \
    {                                                                                                                   \
        cudaError_t e = cudaFuncSetAttribute(scan_tc_kernel<M, O, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)); \
        if (e != cudaSuccess) return e;                                                                                 \
        scan_tc_kernel<M, O, N><<<grid, kThreadsTc, smem, s>>>(p, map, n_slabs, n_qgroups);                             \
    }
    if (onehot) {
        if (nqt == 32) TV_LAUNCH_TC(1, true, 32)
        else if (nqt == 64) TV_LAUNCH_TC(1, true, 64)
        else TV_LAUNCH_TC(1, true, 256)
    } else if (mt == 2) {
        TV_LAUNCH_TC(2, false, 256)
    } else if (nqt == 64) {
        TV_LAUNCH_TC(1, false, 64)
    } else {
        TV_LAUNCH_TC(1, false, 256)
    }
#undef TV_LAUNCH_TC
    return cudaGetLastError();
}

}  // namespace tv
