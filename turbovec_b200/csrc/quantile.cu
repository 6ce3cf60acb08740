// Order statistics of the TQ+ fit on the device.
//
// The fit (encode.rs:737-857) needs, for every coordinate of the rotated sample, the values of two ranks (the
// empirical p_lo and p_hi quantiles).  The sample stays on the device as rows x dim floats; a CTA takes 32 neighbouring
// coordinates (lane = coordinate, so every warp load is one 128-byte line of a row) and finds each rank by a radix
// select over an order-preserving 32-bit key: four passes of 8 bits, each a histogram of the rows whose key matches the
// prefix found so far.  The selected key is the bit pattern of a sample value, so the result is exactly the element an
// exact sort would put at that rank (for equal values any of them; -0.0 and +0.0 compare equal in the reference's
// selection and are 1 apart here, which changes no result because only differences and sums with non-zero terms use them).
#include <cstdint>

#include "ingest.cuh"
#include "tv_common.cuh"

namespace tv {
namespace {

constexpr int kQuantileThreads = 256;
constexpr int kQuantileCoords = 32;
constexpr int kBins = 256;
constexpr int kHistPitch = kBins + 1;                         // lanes of a warp update different coordinates: different banks

__device__ __forceinline__ uint32_t ordered_key(float v) {
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

__global__ void __launch_bounds__(kQuantileThreads)
quantile_pair_kernel(const float *rot, int64_t n, int dim, int64_t lo_rank, int64_t hi_rank, float *q_lo, float *q_hi) {
    __shared__ uint32_t hist[kQuantileCoords * kHistPitch];
    __shared__ uint32_t prefix[kQuantileCoords];
    __shared__ uint32_t remaining[kQuantileCoords];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int coord = blockIdx.x * kQuantileCoords + lane;
    const bool have = coord < dim;
    for (int target = 0; target < 2; ++target) {
        if (tid < kQuantileCoords) { prefix[tid] = 0; remaining[tid] = uint32_t(target == 0 ? lo_rank : hi_rank); }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int i = tid; i < kQuantileCoords * kHistPitch; i += kQuantileThreads) hist[i] = 0;
            __syncthreads();
            const uint32_t want = prefix[lane];
            const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
            if (have) {
                constexpr int kWarps = kQuantileThreads / 32, kUnroll = 8;      // eight row loads in flight per lane
                for (int64_t r0 = warp; r0 < n; r0 += kWarps * kUnroll) {
                    float v[kUnroll];
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) {
                        const int64_t r = r0 + int64_t(u) * kWarps;
                        v[u] = r < n ? __ldg(rot + r * dim + coord) : 0.0f;
                    }
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) {
                        const uint32_t k = ordered_key(v[u]);
                        if (r0 + int64_t(u) * kWarps < n && (k & mask) == want)
                            atomicAdd(&hist[lane * kHistPitch + ((k >> shift) & 0xffu)], 1u);
                    }
                }
            }
            __syncthreads();
            if (tid < kQuantileCoords) {                      // one thread per coordinate walks its 256 bins
                uint32_t rem = remaining[tid], bin = 0;
                const uint32_t *hrow = hist + tid * kHistPitch;
                for (; bin < kBins - 1; ++bin) {
                    const uint32_t c = hrow[bin];
                    if (rem < c) break;
                    rem -= c;
                }
                remaining[tid] = rem;
                prefix[tid] |= bin << shift;
            }
            __syncthreads();
        }
        if (tid < kQuantileCoords && blockIdx.x * kQuantileCoords + tid < dim)
            (target == 0 ? q_lo : q_hi)[blockIdx.x * kQuantileCoords + tid] = key_value(prefix[tid]);
        __syncthreads();
    }
}

}  // namespace

// q_lo[d] / q_hi[d] = the elements of rank lo_rank / hi_rank (0-based, ascending) of column d of rot (n x dim, row-major).
cudaError_t launch_quantile_pair(const float *rot, int64_t n, int dim, int64_t lo_rank, int64_t hi_rank, float *q_lo, float *q_hi,
                                 cudaStream_t stream) {
    if (n <= 0 || dim <= 0) return cudaSuccess;
    if (n > 0xffffffffll) return cudaErrorInvalidValue;       // 32-bit counters
    const unsigned grid = unsigned((dim + kQuantileCoords - 1) / kQuantileCoords);
    quantile_pair_kernel<<<grid, kQuantileThreads, 0, stream>>>(rot, n, dim, lo_rank, hi_rank, q_lo, q_hi);
    return cudaGetLastError();
}

}  // namespace tv
