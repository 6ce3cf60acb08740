// Warp-level implementation of the reference's rotation: two rounds of
// (global permutation with fused sign flip -> Walsh-Hadamard transform of every
// B-coordinate block -> multiply by 1/sqrt(B)), B = largest power-of-two divisor of dim
// (turbovec/src/rotation.rs:28-59, 218-320, 964-982).
//
// Bit-exactness rules followed here: butterflies run in stage order len = 1, 2, 4, ...;
// each output is one rounded add or subtract; the scale is one rounded multiply; nothing is
// fused (explicit __f*_rn intrinsics).  A multiply by a +-1 sign is exact, so it is done as a
// conditional negation.
//
// One warp rotates one row held in shared memory.  A B-block is spread over the warp as
// R = B/32 consecutive coordinates per lane: stages with len < R are register-local, stages
// len = R*m (m = 1..16) exchange registers between lanes `lane` and `lane ^ m`.  For B < 32 a
// lane owns whole blocks; for B > 2048 the transform runs in shared memory.
#pragma once
#include "tv_common.cuh"

namespace tv {

template <int R>
__device__ __forceinline__ void wht_in_registers(float (&v)[R]) {
#pragma unroll
    for (int len = 1; len < R; len <<= 1) {
#pragma unroll
        for (int i = 0; i < R; i += 2 * len) {
#pragma unroll
            for (int j = i; j < i + len; ++j) {
                const float a = v[j], b = v[j + len];
                v[j] = __fadd_rn(a, b);
                v[j + len] = __fsub_rn(a, b);
            }
        }
    }
}

template <int R>
__device__ __forceinline__ void wht_across_lanes(float (&v)[R], int lane) {
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
        const bool upper = (lane & m) != 0;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float other = __shfl_xor_sync(kFullMask, v[r], m);
            // lower element keeps a + b, upper element gets a - b with a = the lower lane's value
            v[r] = upper ? __fsub_rn(other, v[r]) : __fadd_rn(v[r], other);
        }
    }
}

__device__ __forceinline__ float gather_one(const float *src, uint16_t pk, bool use_inv, float inv) {
    float x = src[pk & 0x7fffu];
    if (use_inv) x = __fmul_rn(x, inv);          // (src[perm[i]] * inv) * sign   rotation.rs:384
    return (pk & 0x8000u) ? -x : x;
}

// One round for one row.  src and dst are distinct shared-memory rows of `dim` floats; perm is the
// packed table (low 15 bits source index, bit 15 = negative sign).  LOG2B in 3..11 selects the
// register paths, 12 the shared-memory path (valid for every B).
template <int LOG2B>
__device__ __forceinline__ void rotation_round(const float *src, float *dst, const uint16_t *perm, int dim,
                                               float inv_sqrt_block, bool use_inv, float inv, int lane) {
    if constexpr (LOG2B <= 4) {
        constexpr int B = 1 << LOG2B;
        const int nblk = dim >> LOG2B;
        for (int blk = lane; blk < nblk; blk += 32) {
            float v[B];
#pragma unroll
            for (int r = 0; r < B; ++r) v[r] = gather_one(src, perm[blk * B + r], use_inv, inv);
            wht_in_registers<B>(v);
#pragma unroll
            for (int r = 0; r < B; ++r) dst[blk * B + r] = __fmul_rn(v[r], inv_sqrt_block);
        }
    } else if constexpr (LOG2B <= 11) {
        constexpr int B = 1 << LOG2B;
        constexpr int R = B / 32;
        const int nblk = dim >> LOG2B;
        for (int blk = 0; blk < nblk; ++blk) {
            const int base = blk * B + lane * R;
            float v[R];
#pragma unroll
            for (int r = 0; r < R; ++r) v[r] = gather_one(src, perm[base + r], use_inv, inv);
            wht_in_registers<R>(v);
            wht_across_lanes<R>(v, lane);
#pragma unroll
            for (int r = 0; r < R; ++r) dst[base + r] = __fmul_rn(v[r], inv_sqrt_block);
        }
    } else {
        const int B = dim & -dim;
        for (int i = lane; i < dim; i += 32) dst[i] = gather_one(src, perm[i], use_inv, inv);
        __syncwarp();
        for (int len = 1; len < B; len <<= 1) {
            for (int idx = lane; idx < dim / 2; idx += 32) {
                const int i = (idx / len) * 2 * len + (idx % len);   // blocks are contiguous, B | dim
                const float a = dst[i], b = dst[i + len];
                dst[i] = __fadd_rn(a, b);
                dst[i + len] = __fsub_rn(a, b);
            }
            __syncwarp();
        }
        for (int i = lane; i < dim; i += 32) dst[i] = __fmul_rn(dst[i], inv_sqrt_block);
    }
    __syncwarp();
}

// Both rounds: row -> tmp -> row.  With use_inv the first gather multiplies by `inv` first
// (Rotation::apply_scaled_into, rotation.rs:218-256); without it this is Rotation::apply
// (rotation.rs:265-320), the query-side form.
template <int LOG2B>
__device__ __forceinline__ void rotate_row(float *row, float *tmp, const uint16_t *perm0, const uint16_t *perm1,
                                           int dim, float inv_sqrt_block, bool use_inv, float inv, int lane) {
    rotation_round<LOG2B>(row, tmp, perm0, dim, inv_sqrt_block, use_inv, inv, lane);
    rotation_round<LOG2B>(tmp, row, perm1, dim, inv_sqrt_block, false, 1.0f, lane);
}

// Template selector: log2 of the block size, clamped to 12 (= shared-memory path).
inline int rotation_variant(int dim) {
    int b = dim & -dim, l = 0;
    while ((1 << l) < b) ++l;
    return l > 11 ? 12 : l;
}

}  // namespace tv
