// Device-side helpers shared by the scan kernels on CUDA-core MMAs (search.cu, scan_small.cu): candidate push,
// mbarrier and bulk-copy wrappers (every wait bounded), byte permutes, the transposing matrix load and the warp-level
// int8 MMA, and the level lookups of the permute-dot family.
#pragma once
#include "search.cuh"
#include "tv_common.cuh"

namespace tv {
namespace {

constexpr int kLanes = 32;   // vectors per code block

// =====================================================================================================
// Candidate push shared by the scan kernels
// =====================================================================================================
__device__ __forceinline__ void push_candidate(const CandidateBuffers &cb, int q, float score, uint32_t slot,
                                               uint64_t thr, uint64_t lo = 0) {
    const uint64_t key = make_key(score, slot);
    if (key < thr && key >= lo) {
        const uint32_t pos = atomicAdd(&cb.cnt[q], 1u);
        if (pos < uint32_t(cb.cap)) cb.cand[size_t(q) * cb.cap + pos] = key;
    }
}

// =====================================================================================================
// PTX helpers: mbarrier + bulk asynchronous copy (no multicast), warp-level int8 MMA
// =====================================================================================================
__device__ __forceinline__ uint32_t smem_addr(const void *p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after kWaitLimit polls (each poll itself blocks for a hardware-defined
// interval), records the failure and lets the caller leave its loop.
constexpr uint32_t kWaitLimit = 1u << 22;
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t *error_flag) {
    for (uint32_t i = 0; i < kWaitLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(error_flag, 1u);
    return false;
}
__device__ __forceinline__ void bulk_copy_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(dst)),
                 "l"(src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// Two 16 x 16 byte matrices, transposed by the load unit: lane 4*q + t receives in x[2*i + h] the bytes of column
// q + 8*h of matrix i from its rows 4t .. 4t+3 (byte r of the word = row 4t + r).  Lanes 0..15 give the row
// addresses of matrix 0, lanes 16..31 those of matrix 1 (16-byte aligned, 16 bytes each).
__device__ __forceinline__ void ldmatrix_x2_trans_b8(uint32_t (&x)[4], uint32_t row_addr) {
    asm volatile("ldmatrix.sync.aligned.m16n16.x2.trans.shared.b8 {%0, %1, %2, %3}, [%4];"
                 : "=r"(x[0]), "=r"(x[1]), "=r"(x[2]), "=r"(x[3])
                 : "r"(row_addr)
                 : "memory");
}
__device__ __forceinline__ void mma_s8(int (&c)[4], const uint4 &a, uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
}

// high 32 bits of a * b + c on the FMA pipe: a right shift that does not load the (saturated) ALU pipe
__device__ __forceinline__ uint32_t mad_hi(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("mad.hi.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ void expand4(uint32_t x, const uint32_t (&T)[4], uint32_t &b0, uint32_t &b1) {
    const uint32_t idx = x & 0x77777777u;                     // low three bits of every nibble
    // byte i from the low or the high half-table: nibble i = i + 4 * (bit 3 of code i); (x & 8..8) >> 1 + 0x3210..
    const uint32_t pick = mad_hi(x & 0x88888888u, 0x80000000u, 0x32103210u);
    b0 = prmt(prmt(T[0], T[1], idx), prmt(T[2], T[3], idx), pick);
    const uint32_t idx_h = mad_hi(idx, 0x10000u, 0u), pick_h = mad_hi(pick, 0x10000u, 0u);   // >> 16
    b1 = prmt(prmt(T[0], T[1], idx_h), prmt(T[2], T[3], idx_h), pick_h);
}

// Split lookup for a codebook whose levels 0..7 are <= 0 and 8..15 are >= 0 (every Lloyd-Max codebook of the
// reference is symmetric).  A packed nibble is a `prmt` selector as it stands: values 0..7 pick a byte of the
// 8-byte table, values 8..15 ask for the sign of that byte replicated - 0x00 when the table holds
// non-negative bytes.  So `prmt(Tn, x)` yields -level[c] where c < 8 and 0 elsewhere, `prmt(Tp, x ^ 8..8)`
// yields level[c] where c >= 8 and 0 elsewhere, with no masking and no merge: S = W.pos - W.neg, both exact
// int32 contractions.  Five ALU-pipe operations per eight codes against eight in expand4; the second MMA is
// paid by the tensor pipe, which this scan leaves mostly idle.
__device__ __forceinline__ void expand4_split(uint32_t x, const uint32_t (&Tp)[2], const uint32_t (&Tn)[2], uint32_t &p0,
                                              uint32_t &p1, uint32_t &n0, uint32_t &n1) {
    const uint32_t y = x ^ 0x88888888u;
    const uint32_t xh = mad_hi(x, 0x10000u, 0u), yh = mad_hi(y, 0x10000u, 0u);   // >> 16 on the FMA pipe
    n0 = prmt(Tn[0], Tn[1], x);
    p0 = prmt(Tp[0], Tp[1], y);
    n1 = prmt(Tn[0], Tn[1], xh);
    p1 = prmt(Tp[0], Tp[1], yh);
}
__host__ __device__ inline uint32_t negate_bytes(uint32_t w) {                   // per-byte two's complement
    uint32_t r = 0;
    for (int b = 0; b < 4; ++b) r |= uint32_t(uint8_t(-int(int8_t(w >> (8 * b))))) << (8 * b);
    return r;
}
// whether the level table allows the split lookup
inline bool levels_split_ok(const uint32_t (&words)[4]) {
    for (int c = 0; c < 16; ++c) {
        const int v = int8_t(words[c / 4] >> (8 * (c % 4)));
        if (c < 8 ? (v > 0 || v == -128) : v < 0) return false;
    }
    return true;
}

}  // namespace
}  // namespace tv
