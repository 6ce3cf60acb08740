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
// One warp rotates one row held in shared memory.  Coordinate e of a B-block sits in lane e % 32,
// register e / 32: consecutive lanes touch consecutive shared-memory words (no bank conflicts), stages
// len < 32 exchange values between lanes `lane` and `lane ^ len`, stages len >= 32 pair registers — the
// stage order stays len = 1, 2, 4, ...  For B < 32 several blocks share a warp pass; for B > 2048 the
// transform runs in shared memory.
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

// Stages len = 1 .. MAXLEN/2 between lanes: the lane with bit `len` clear holds the lower element.
template <int R, int MAXLEN>
__device__ __forceinline__ void wht_across_lanes(float (&v)[R], int lane) {
#pragma unroll
    for (int m = 1; m < MAXLEN; m <<= 1) {
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
        // 32 / B whole blocks per pass of the warp; B divides 32 and dim, so a ragged last pass still
        // holds whole blocks and the idle lanes only feed shuffles nobody reads
        constexpr int B = 1 << LOG2B;
        for (int base = 0; base < dim; base += 32) {
            const int idx = base + lane;
            const bool active = idx < dim;
            float v[1] = {active ? gather_one(src, perm[idx], use_inv, inv) : 0.0f};
            wht_across_lanes<1, B>(v, lane);
            if (active) dst[idx] = __fmul_rn(v[0], inv_sqrt_block);
        }
    } else if constexpr (LOG2B <= 11) {
        constexpr int B = 1 << LOG2B;
        constexpr int R = B / 32;
        const int nblk = dim >> LOG2B;
        for (int blk = 0; blk < nblk; ++blk) {
            const int base = blk * B + lane;
            float v[R];
#pragma unroll
            for (int r = 0; r < R; ++r) v[r] = gather_one(src, perm[base + r * 32], use_inv, inv);
            wht_across_lanes<R, 32>(v, lane);     // len = 1 .. 16
            wht_in_registers<R>(v);               // len = 32 .. B/2 (register r holds coordinates r*32 + lane)
#pragma unroll
            for (int r = 0; r < R; ++r) dst[base + r * 32] = __fmul_rn(v[r], inv_sqrt_block);
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
