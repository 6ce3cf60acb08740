// Device-side pieces shared by the tensor-memory scans (scan_tc.cu, scan_tc_wide.cu, scan_tc_dense.cu, scan_tc_dense2.cu):
// constants of the MMA tiling, bounded mbarrier waits, the nibble -> int8 level lookup, shared-memory and
// instruction descriptors, TMA and TMEM wrappers, and the float epilogue of the score families.
#pragma once
#include <cuda.h>

#include <climits>
#include <cstddef>

#include "search.cuh"
#include "tv_common.cuh"

namespace tv {
namespace {

constexpr int kMmaM = 128;                                    // vectors per accumulator tile (TMEM lanes)
constexpr int kMaxTileQueries = 256;                          // largest MMA N (query columns of a work item)
constexpr int kSlabK = 128;                                   // int8 elements (bytes) of K per stage
constexpr int kATileBytes = kMmaM * kSlabK;                   // 16 KB per accumulator tile and stage
constexpr int kExpandWarps = 8;
constexpr int kEpilogueWarps = 8;                             // two per TMEM lane quarter, 128 columns each
constexpr int kThreadsTc = (2 + kEpilogueWarps + kExpandWarps) * 32;   // 576
constexpr uint32_t kWaitLimitTc = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t *error_flag) {
    for (uint32_t i = 0; i < kWaitLimitTc; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(error_flag, 2u);
    return false;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// high 32 bits of a * b + c on the FMA pipe: a right shift that does not load the ALU pipe
__device__ __forceinline__ uint32_t mad_hi(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("mad.hi.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// Eight nibbles of x -> eight int8 levels; output byte i of (lo, hi) belongs to nibble i / i+4 of x.
__device__ __forceinline__ void expand8(uint32_t x, const uint32_t (&T)[4], uint32_t &lo, uint32_t &hi) {
    const uint32_t idx = x & 0x77777777u;
    const uint32_t pick = mad_hi(x & 0x88888888u, 0x80000000u, 0x32103210u);   // ((x >> 1) & 0x4..4) | 0x3210..
    lo = prmt(prmt(T[0], T[1], idx), prmt(T[2], T[3], idx), pick);
    const uint32_t idx_h = mad_hi(idx, 0x10000u, 0u), pick_h = mad_hi(pick, 0x10000u, 0u);
    hi = prmt(prmt(T[0], T[1], idx_h), prmt(T[2], T[3], idx_h), pick_h);
}

// K-major, 128-byte swizzle, 8-row groups 1024 B apart; version 1 (sm_100), base offset 0.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_byte_addr) {
    uint64_t d = 0;
    d |= uint64_t((smem_byte_addr >> 4) & 0x3fffu);           // start address
    d |= uint64_t(1) << 16;                                    // leading byte offset (unused for swizzled K-major)
    d |= uint64_t(1024 >> 4) << 32;                            // stride byte offset
    d |= uint64_t(1) << 46;                                    // descriptor version
    d |= uint64_t(2) << 61;                                    // SWIZZLE_128B
    return d;
}
// kind::i8: D = S32, A = B = signed 8-bit, both K-major, M = 128, N = NQT.
template <int NQT>
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(NQT >> 3) << 17) | (uint32_t(kMmaM >> 4) << 24);
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kIdesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}

// ---- CTA pairs (clusters of two, tcgen05 cta_group::2): scan_tc_dense2.cu ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Remote arrivals carry the default (CTA-scope release) semantics: what they publish was written to the arriving CTA's own
// shared memory and made visible to the asynchronous proxy by fence.proxy.async before the arrival; a cluster-scope
// release on every arrival cost more than the MMAs it guarded.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t *bar, uint32_t parity, uint32_t *error_flag) {
    for (uint32_t i = 0; i < kWaitLimitTc; ++i)
        if (mbar_try_wait_cluster(bar, parity)) return true;
    atomicExch(error_flag, 3u);
    return false;
}
// kind::i8 across the pair: D = S32, A = B = signed 8-bit, both K-major, M = 256 (128 rows per CTA), N = 256.
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(256 >> 3) << 17) | (uint32_t(256 >> 4) << 24);
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kIdesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// arrives on the barrier at `cluster_addr` (this CTA's or the peer's) once the pair's MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}
// this CTA's half of a query slab; the transaction bytes are reported to the leader's barrier
__device__ __forceinline__ void tma_load_2d_pair(void *dst, const CUtensorMap *map, int x, int y, uint32_t leader_bar_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(leader_bar_addr), "r"(x), "r"(y) : "memory");
}

// Float epilogue of the score families; the integer sum is exact in all of them.  Permute-dot: fma((f32)S, scale, bias)
// (search.rs:1523, 1793).  u8-LUT, mul-add family: (f32)isum * scale + bias (search.rs:1176).  u8-LUT, flush family
// with at most 256 byte-groups (`fused`): one fma(scale, (f32)isum, bias) (search.rs:516, 577, 1596) - the same
// single rounding as the permute-dot form.  Then x vec_scale.
template <bool ONEHOT>
__device__ __forceinline__ float final_score(bool fused, uint32_t isum, float qs, float qb, float vs) {
    const float f = float(int(isum));
    if constexpr (ONEHOT) return __fmul_rn(fused ? fmaf(qs, f, qb) : __fadd_rn(__fmul_rn(f, qs), qb), vs);
    else return __fmul_rn(fmaf(f, qs, qb), vs);
}


// Integer bound that dismisses most accumulator columns without converting them to float.
// For one query (scale qs > 0, bias qb, threshold score t > 0) and every vector of a work item (vector scales
// 0 <= vs <= vs_max), a score fmul(fma((f32)isum, qs, qb), vs) can reach t only if
//     isum >= ((t / vs_max) - qb) / qs
// up to the roundings of the conversion, the fma and the multiply (each within 2^-23 relative).  The returned integer
// lies below that bound by a margin a thousand times those roundings plus two units, so `isum >= bound` is necessary
// for a candidate; the columns that satisfy it are scored exactly afterwards.  The integer compare costs one
// instruction per column where the exact score costs four, one of them (int -> float) on a quarter-rate unit; on
// L2-normalised data the vector scales of an item differ by a few percent, so hardly any column survives it.
// t <= 0 (no k-th result yet, or a non-positive one): everything is kept.  vs_max = 0 with t > 0: nothing can pass.
__device__ __forceinline__ int dismissal_bound(float qs, float qb, float t, float vs_max) {
    if (!(t > 0.0f)) return INT_MIN;
    if (!(qs > 0.0f)) return qb * vs_max >= t ? INT_MIN : INT_MAX;     // a column without a query has t = +inf
    const float g = t / vs_max;                                        // +inf when vs_max is 0
    const float bound = (g - qb) / qs;
    const float margin = 1.0e-5f * (fabsf(g) + fabsf(qb)) / qs + 2.0f;
    const float lo = bound - margin;
    if (!(lo < 2.0e9f)) return INT_MAX;
    if (lo < -2.0e9f) return INT_MIN;
    return __float2int_rd(lo);
}


// First chunk of an unfiltered search: the 32 accumulator columns of a piece (queries ql0 .. ql0 + 31 of one vector) go to
// position `at` of their queries' candidate lists, every one of them.  qscale / qbias point at the piece's first column.
template <bool ONEHOT>
__device__ __forceinline__ void write_piece(const uint32_t (&acc)[32], const float *qscale, const float *qbias, bool fused, float vs,
                                            bool live, int64_t slot, int ql0, int nq_end, uint32_t at, const CandidateBuffers &cb) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const int ql = ql0 + j;
        if (ql < nq_end) {
            const float score = final_score<ONEHOT>(fused, acc[j], qscale[j], qbias[j], vs);
            cb.cand[size_t(ql) * cb.cap + at] = live ? make_key(score, uint32_t(slot)) : kEmptyKey;
        }
    }
}

// Later chunks: one integer compare per column dismisses the piece unless some column could be a candidate
// (dismissal_bound).  Each lane keeps the outcome per run of 8 columns; the runs that any lane of the warp flagged are
// re-read from tensor memory (address `taddr` = the piece's first column) and scored exactly by the lanes that flagged
// them, and the keys that beat the query's k-th key are appended to its candidate list.  All pointers are at the
// piece's first column; every lane of the warp must call this.
template <bool ONEHOT>
__device__ __forceinline__ void sift_piece(const uint32_t (&acc)[32], const int *ibound, const float *qscale, const float *qbias,
                                           const float *qthr, bool fused, float vs, bool live, int64_t slot, int ql0, uint32_t taddr,
                                           const CandidateBuffers &cb) {
    uint32_t runs = 0;
    const int4 *pi = reinterpret_cast<const int4 *>(ibound);
#pragma unroll
    for (int j4 = 0; j4 < 8; ++j4) {
        const int4 b = pi[j4];
        const bool may = (int(acc[4 * j4 + 0]) >= b.x) | (int(acc[4 * j4 + 1]) >= b.y) | (int(acc[4 * j4 + 2]) >= b.z) |
                         (int(acc[4 * j4 + 3]) >= b.w);
        runs |= uint32_t(may) << (j4 >> 1);
    }
    if (!live) runs = 0;
    const uint32_t warp_runs = __reduce_or_sync(0xffffffffu, runs);
    if (warp_runs == 0) return;
#pragma unroll 1
    for (int c1 = 0; c1 < 32; c1 += 8) {
        if (!((warp_runs >> (c1 >> 3)) & 1u)) continue;
        uint32_t a8[8];
        tmem_ld8(taddr + c1, a8);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if ((runs >> (c1 >> 3)) & 1u) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int c = c1 + e;
                const float score = final_score<ONEHOT>(fused, a8[e], qscale[c], qbias[c], vs);
                if (score >= qthr[c]) {
                    const int ql = ql0 + c;
                    const uint64_t key = make_key(score, uint32_t(slot));
                    if (key < cb.thr[ql] && (cb.lo == nullptr || key >= cb.lo[ql])) {
                        const uint32_t at = atomicAdd(&cb.cnt[ql], 1u);
                        if (at < uint32_t(cb.cap)) cb.cand[size_t(ql) * cb.cap + at] = key;
                    }
                }
            }
        }
    }
}

}  // namespace
}  // namespace tv
