// Shared device-side helpers and launch plumbing for the turbovec_b200 kernels.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

namespace tv {

constexpr unsigned kFullMask = 0xffffffffu;

// Result ordering.  The reference orders results by (score descending, slot ascending)
// (turbovec/src/search.rs:236-252, 4285-4290).  Every (score, slot) pair is mapped to one u64 key
// whose ASCENDING order is that total order: high word = bit-flipped order-preserving image of the
// f32 score, low word = slot.  -0.0 is folded onto +0.0 first because the reference compares scores
// with partial_cmp, under which the two zeros tie.
__host__ __device__ inline uint32_t score_to_desc_bits(float s) {
    if (s == 0.0f) s = 0.0f;
#ifdef __CUDA_ARCH__
    uint32_t u = __float_as_uint(s);
#else
    union { float f; uint32_t u; } cvt; cvt.f = s; uint32_t u = cvt.u;
#endif
    uint32_t asc = (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // ascending in s
    return ~asc;                                                  // descending in s
}
__host__ __device__ inline float desc_bits_to_score(uint32_t d) {
    uint32_t asc = ~d;
    uint32_t u = (asc & 0x80000000u) ? (asc & 0x7fffffffu) : ~asc;
#ifdef __CUDA_ARCH__
    return __uint_as_float(u);
#else
    union { float f; uint32_t u; } cvt; cvt.u = u; return cvt.f;
#endif
}
__host__ __device__ inline uint64_t make_key(float score, uint32_t slot) {
    return (uint64_t(score_to_desc_bits(score)) << 32) | slot;
}
constexpr uint64_t kEmptyKey = 0xffffffffffffffffull;   // sorts after every real key; "no result yet"

}  // namespace tv
