// Pipelined ingest kernel for whole 32-slot code blocks of an uncalibrated index: the same arithmetic as
// ingest.cu (encode::encode, turbovec/src/encode.rs:510-541 = rotate_batch_into :406-458 + encode_prerotated
// :560-652 / fused_quantize_scale_pack_scalar :1418-1476, blocked layout pack.rs:340-361), reorganised so
// that the order-fixed sequential sums no longer stall the data-parallel work.
//
// One CTA of three warpgroups walks a contiguous range of code blocks in waves of 8 vectors and runs its
// stages concurrently, one wave apart, with one CTA barrier per step:
//   norm warp      wave i     8 sequential f32 chains per vector straight from global memory (4 lanes per
//                             vector, two chains per lane), fixed combine tree, sqrt, reciprocal
//   8 rotation     wave i-1   one warp per vector, the whole vector in registers: both rounds of permutation,
//   warps                     sign flip and Walsh-Hadamard butterflies (rotation.cuh states the order rules),
//                             Lloyd-Max quantisation by a register binary search, packing into the block tile
//   sum warp       wave i-2   4 sequential f64 chains per vector over the rotated row and the codes, scale;
//                             then issues the bulk copies that stage wave i's rows into shared memory
//   2 copy warps              write the finished tile of a block (ngroups x 32 bytes, word-swizzled so that the
//                             byte stores of a warp never share a bank) to the code array
// Rows arrive by cp.async.bulk with an mbarrier transaction count.  The two rotation warpgroups take the
// registers the third one gives up (setmaxnreg), so a 2048-coordinate vector and its permutation entries
// stay in registers.
#include <algorithm>
#include <cmath>

#include "ingest.cuh"
#include "tv_common.cuh"

namespace tv {
namespace {

constexpr uint32_t kWaitLimitIngest = 1u << 26;   // mbarrier polls before a wait gives up

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
    for (uint32_t i = 0; i < kWaitLimitIngest; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(error_flag, 3u);
    return false;
}
// global -> shared bulk copy; both addresses 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// shared-memory accesses by 32-bit shared address: keeps the address arithmetic of the fully unrolled
// rotation in one register per access
__device__ __forceinline__ float lds_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts_f32(uint32_t addr, float v) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void sts_u8(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.u8 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ float max_nan(float a, float b) {   // NaN wins, unlike fmaxf
    float d;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
    return d;
}

constexpr int kWave = 8;                 // vectors per wave = rotation warps
constexpr int kWavesPerBlock = kBlockLanes / kWave;
constexpr int kFastThreads = 384;        // 8 rotation warps, norm warp, sum warp, 2 copy warps
constexpr int kRotationRegs = 208, kServiceRegs = 88;   // 8*32*208 + 4*32*88 <= 384 * 168

struct FastLayout {
    int stride;          // floats per staged row: dim + 4 keeps the sum warp's 4-lane reads on distinct banks
    size_t rows, tile, table, norm, inv, bars, total;
};
__host__ __device__ inline FastLayout fast_layout(int dim, int ngroups, int cpb) {
    FastLayout L;
    L.stride = dim + 4;
    size_t off = 0;
    L.rows = off; off += size_t(2) * kWave * L.stride * 4;
    L.tile = off; off += size_t(2) * ngroups * 32;
    L.table = off; off += size_t(cpb) * 256 * 8;     // centroid (as f64) of field k of every byte value
    L.norm = off; off += 3 * kWave * 4;
    L.inv = off; off += 3 * kWave * 4;
    L.bars = off; off += 2 * 8;
    L.total = off;
    return L;
}

// Register binary search: number of boundaries strictly below x (encode.rs:1447-1451).  b holds the
// boundaries of a 2-, 3- or 4-bit codebook padded to 15 entries with +inf, which steers the upper levels
// of the search into the populated part.
struct Boundaries15 { float b[15]; };   // passed by value: the search then takes them as constant-bank operands
__device__ __forceinline__ uint32_t quantise15(float x, const float (&b)[15]) {
    const bool p1 = x > b[7];
    const bool p2 = x > (p1 ? b[11] : b[3]);
    const float u0 = p2 ? b[5] : b[1], u1 = p2 ? b[13] : b[9];
    const bool p3 = x > (p1 ? u1 : u0);
    const float w0 = p3 ? b[2] : b[0], w1 = p3 ? b[6] : b[4], w2 = p3 ? b[10] : b[8], w3 = p3 ? b[14] : b[12];
    const float y0 = p2 ? w1 : w0, y1 = p2 ? w3 : w2;
    const bool p4 = x > (p1 ? y1 : y0);
    return (p1 ? 8u : 0u) + (p2 ? 4u : 0u) + (p3 ? 2u : 0u) + (p4 ? 1u : 0u);
}

// Walsh-Hadamard transform of NBLK blocks of 32*R coordinates; v[b*R + r] holds coordinate r*32 + lane of
// block b.  Stage order len = 1, 2, 4, ...: lane exchanges first, register pairs after.  fma(v, +-1, other)
// rounds once, exactly like the add or subtract it stands for.
template <int R, int NBLK>
__device__ __forceinline__ void wht_blocks(float (&v)[R * NBLK], const float (&sgn)[5]) {
#pragma unroll
    for (int s = 0; s < 5; ++s) {
#pragma unroll
        for (int k = 0; k < R * NBLK; ++k) {
            const float other = __shfl_xor_sync(kFullMask, v[k], 1 << s);
            v[k] = __fmaf_rn(v[k], sgn[s], other);   // lower lane: v + other; upper lane: other - v
        }
    }
#pragma unroll
    for (int len = 1; len < R; len <<= 1) {
#pragma unroll
        for (int b = 0; b < NBLK; ++b) {
#pragma unroll
            for (int i = 0; i < R; i += 2 * len) {
#pragma unroll
                for (int j = i; j < i + len; ++j) {
                    const float x = v[b * R + j], y = v[b * R + j + len];
                    v[b * R + j] = __fadd_rn(x, y);
                    v[b * R + j + len] = __fsub_rn(x, y);
                }
            }
        }
    }
}

// The 4 sequential f64 chains of 8 vectors: lane = (vector vv, chain c), chain c sums
// rotated[j] * centroid[code[j]] over j = c (mod 4) in ascending j (encode.rs:1418-1476).  `tab` maps a
// tile byte straight to the centroid of this chain's field; the word swizzle of the tile repeats every 32
// groups, so inside a window of 32 groups every offset is a compile-time constant.
template <int CPB, int DIM>
__device__ __forceinline__ double sum_chain(const float *row_c, const unsigned char *tile_lane, int wsel, const double *tab) {
    constexpr int GS = 4 / CPB;                 // groups advanced per step
    constexpr int SW = 32 / GS;                 // steps per window of 32 groups
    const unsigned char *ps[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) ps[s] = tile_lane + (((wsel ^ s) & 7) << 2);
    double acc = 0.0;
#pragma unroll 1
    for (int wnd = 0; wnd < DIM / 4 / SW; ++wnd) {
#pragma unroll
        for (int u = 0; u < SW; ++u) {
            const uint32_t byte = ps[((GS * u) >> 2) & 7][GS * u * 32];
            acc = __dadd_rn(acc, __dmul_rn(double(row_c[4 * u]), tab[byte]));
        }
#pragma unroll
        for (int s = 0; s < 8; ++s) ps[s] += 1024;
        row_c += 4 * SW;
    }
    return acc;
}

template <int LOG2B, int NBLK>
__global__ void __launch_bounds__(kFastThreads, 1) ingest_fast_kernel(IngestParams p, Boundaries15 bnd, uint32_t *error) {
    constexpr int R = 1 << (LOG2B - 5);               // registers per Hadamard block and lane
    constexpr int T = R * NBLK;                       // registers per vector and lane
    constexpr int DIM = T * 32;
    constexpr int V = kWave, wpb = kWavesPerBlock;
    static_assert(T % 4 == 0, "the packing below handles whole groups of four registers");
    extern __shared__ __align__(128) unsigned char smem[];
    const int ng = p.ngroups;
    const int cpb = p.bits == 2 ? 4 : 2;              // codes per byte (3-bit codes sit in 4-bit fields)
    const int field = 8 / cpb;
    const FastLayout L = fast_layout(DIM, ng, cpb);
    float *rows = reinterpret_cast<float *>(smem + L.rows);
    unsigned char *tiles = smem + L.tile;
    double *table = reinterpret_cast<double *>(smem + L.table);   // [cpb][256]
    float *norm_s = reinterpret_cast<float *>(smem + L.norm);     // [3][8]
    float *inv_s = reinterpret_cast<float *>(smem + L.inv);       // [3][8]
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + L.bars); // [2]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int stride = L.stride;
    const int tile_bytes = ng * 32;

    const int64_t slot_lo = p.slot0, slot_hi = p.slot0 + p.n;       // slot_lo is a multiple of 32
    const int64_t nblocks = (p.n + 31) / 32;
    const int64_t b0 = nblocks * blockIdx.x / gridDim.x, b1 = nblocks * (blockIdx.x + 1) / gridDim.x;
    const int nw = int(b1 - b0) * wpb;                // waves of this CTA
    const int64_t first_block = slot_lo / 32 + b0;

    if (tid == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = tid; i < cpb * 256; i += kFastThreads) {
        const int k = i >> 8, byte = i & 255;
        table[i] = double(p.centroids[(byte >> ((cpb - 1 - k) * field)) & ((1 << field) - 1)]);   // the codebook array has 16 slots
    }
    __syncthreads();

    // slot of vector `v` of wave `w`, or -1 past the new rows (padding lanes of the last block)
    auto wave_slot = [&](int w, int v) -> int64_t {
        const int64_t s = (first_block + w / wpb) * 32 + (w % wpb) * V + v;
        return s < slot_hi ? s : -1;
    };

    if (warp < V) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRotationRegs) : "memory");
        // ------------------------------------------------ rotation + quantisation: one vector per warp
        uint32_t pk[T];          // per register: round-1 byte offset | sign << 15, round-2 the same in the high half
#pragma unroll
        for (int k = 0; k < T; ++k) {
            const uint32_t e0 = p.perm0[k * 32 + lane], e1 = p.perm1[k * 32 + lane];
            pk[k] = ((e0 & 0x7fffu) << 2) | (e0 & 0x8000u) | ((((e1 & 0x7fffu) << 2) | (e1 & 0x8000u)) << 16);
        }
        float sgn[5];
#pragma unroll
        for (int s = 0; s < 5; ++s) sgn[s] = (lane >> s) & 1 ? -1.0f : 1.0f;
        const float isb = p.inv_sqrt_block;
        const int q = lane & (cpb - 1);               // this lane packs the registers k = q (mod cpb)

        for (int it = 0; it <= nw + 1; ++it) {
            const int w = it - 1;
            if (w >= 0 && w < nw) {
                const int64_t slot = wave_slot(w, warp);
                uint32_t cw[(T + 7) / 8];             // 4-bit code of register k in nibble k % 8 of word k / 8
#pragma unroll
                for (int i = 0; i < (T + 7) / 8; ++i) cw[i] = 0;
                float *row = rows + size_t((w & 1) * V + warp) * stride;
                if (slot >= 0 && mbar_wait(&full[w & 1], (w >> 1) & 1, error)) {
                    const uint32_t rb = smem_u32(row), rl = rb + lane * 4;
                    const float inv = inv_s[(w % 3) * V + warp];
                    // keeps the masks and offsets derived from pk from being hoisted out of the wave loop into
                    // four registers per entry
#pragma unroll
                    for (int k = 0; k < T; ++k) asm volatile("" : "+r"(pk[k]));
                    float v[T];
                    // round 1: (x[perm] * inv) * sign (rotation.rs:384); |x| < 1e16 checked on the way (encode.rs:58-74)
                    float big = 0.0f;
#pragma unroll
                    for (int k = 0; k < T; ++k) {
                        const float x = lds_f32(rb + (pk[k] & 0x7ffcu));
                        big = max_nan(big, fabsf(x));
                        v[k] = __uint_as_float(__float_as_uint(__fmul_rn(x, inv)) ^ ((pk[k] << 16) & 0x80000000u));
                    }
                    __syncwarp();
                    if (__any_sync(kFullMask, !(big < kMaxMagnitude))) {
                        const int64_t r = slot - slot_lo;
                        for (int j = lane; j < DIM; j += 32)
                            if (!(fabsf(row[j]) < kMaxMagnitude))
                                atomicMin(p.first_invalid, (unsigned long long)((p.row_base + r) * DIM + j));
                        __syncwarp();
                    }
                    wht_blocks<R, NBLK>(v, sgn);
#pragma unroll
                    for (int k = 0; k < T; ++k) sts_f32(rl + k * 128, __fmul_rn(v[k], isb));
                    __syncwarp();
                    // round 2
#pragma unroll
                    for (int k = 0; k < T; ++k) {
                        const float x = lds_f32(rb + ((pk[k] >> 16) & 0x7ffcu));
                        v[k] = __uint_as_float(__float_as_uint(x) ^ (pk[k] & 0x80000000u));
                    }
                    __syncwarp();
                    wht_blocks<R, NBLK>(v, sgn);
#pragma unroll
                    for (int k = 0; k < T; ++k) {
                        const float y = __fmul_rn(v[k], isb);
                        sts_f32(rl + k * 128, y);                     // rotated row, read by the sum warp
                        cw[k >> 3] |= quantise15(y, bnd.b) << (4 * (k & 7));
                    }
                }
                // pack: byte of group g = codes of coordinates g*cpb .. g*cpb+cpb-1, first one in the top field
                // (pack.rs:264-282); the cpb lanes of a group exchange code words, lane q stores k = q (mod cpb)
                const int vabs = (w % wpb) * V + warp;                // lane of this vector in its block
                const uint32_t tile = smem_u32(tiles) + ((w / wpb) & 1) * tile_bytes;
                if (cpb == 2) {
                    const uint32_t dst = tile + q * 512 + (lane >> 1) * 32 + ((((vabs >> 2) ^ (4 * q + (lane >> 3))) & 7) << 2) + (vabs & 3);
#pragma unroll
                    for (int wd = 0; wd < (T + 7) / 8; ++wd) {
                        const uint32_t other = __shfl_xor_sync(kFullMask, cw[wd], 1);
                        const uint32_t ev = q ? other : cw[wd], od = q ? cw[wd] : other;
                        const uint32_t bytes = (((ev >> (4 * q)) & 0x0f0f0f0fu) << 4) | ((od >> (4 * q)) & 0x0f0f0f0fu);
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (8 * wd + 2 * i < T) sts_u8(dst + (8 * wd + 2 * i) * 512, bytes >> (8 * i));
                    }
                } else {
                    const uint32_t dst = tile + q * 256 + (lane >> 2) * 32 + ((((vabs >> 2) ^ (2 * q + (lane >> 4))) & 7) << 2) + (vabs & 3);
#pragma unroll
                    for (int wd = 0; wd < (T + 7) / 8; ++wd) {
                        uint32_t bytes = 0;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t xj = __shfl_sync(kFullMask, cw[wd], (lane & ~3) + j);
                            bytes |= ((xj >> (4 * q)) & 0x00030003u) << (6 - 2 * j);
                        }
                        sts_u8(dst + (8 * wd) * 256, bytes);
                        if (8 * wd + 4 < T) sts_u8(dst + (8 * wd + 4) * 256, bytes >> 16);
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncthreads();
        }
    } else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kServiceRegs) : "memory");
        if (warp == V) {
            // -------------------------------------------- norms, one wave ahead of the rotation
            const int vv = lane >> 2, pp = lane & 3;
            for (int it = 0; it <= nw + 1; ++it) {
                if (it + 1 < nw && lane < V) {
                    // pull the rows of the next wave into L2: this warp reads them in the next step, the
                    // bulk copies one step later
                    const int64_t slot = wave_slot(it + 1, lane);
                    if (slot >= 0)
                        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.x + (slot - slot_lo) * DIM), "r"(DIM * 4) : "memory");
                }
                if (it < nw) {
                    const int64_t slot = wave_slot(it, vv);
                    float a0 = 0.0f, a1 = 0.0f;
                    if (slot >= 0) {
                        // chains 2pp and 2pp+1: x[j]^2 summed over j = chain (mod 8) in ascending j (encode.rs:900-932)
                        const float2 *src = reinterpret_cast<const float2 *>(p.x + (slot - slot_lo) * DIM + 2 * pp);
#pragma unroll 1
                        for (int t0 = 0; t0 < DIM / 8; t0 += 16) {
                            float2 x[16];
#pragma unroll
                            for (int u = 0; u < 16; ++u) x[u] = __ldg(src + 4 * (t0 + u));
#pragma unroll
                            for (int u = 0; u < 16; ++u) {
                                a0 = __fadd_rn(a0, __fmul_rn(x[u].x, x[u].x));
                                a1 = __fadd_rn(a1, __fmul_rn(x[u].y, x[u].y));
                            }
                        }
                    }
                    float s = __fadd_rn(a0, a1);                                  // (c0+c1), (c2+c3), (c4+c5), (c6+c7)
                    s = __fadd_rn(s, __shfl_down_sync(kFullMask, s, 1));          // valid on pp = 0 and pp = 2
                    s = __fadd_rn(s, __shfl_down_sync(kFullMask, s, 2));          // valid on pp = 0
                    if (pp == 0) {
                        const float nv = __fsqrt_rn(s);
                        norm_s[(it % 3) * V + vv] = nv;
                        inv_s[(it % 3) * V + vv] = nv > kMinNorm ? __fdiv_rn(1.0f, nv) : 0.0f;    // encode.rs:446
                    }
                }
                __syncthreads();
            }
        } else if (warp == V + 1) {
            // -------------------------------------------- reconstruction sums two waves behind; row staging
            const int vv = lane >> 2, c = lane & 3;
            const double *tab = table + (c % cpb) * 256;
            for (int it = 0; it <= nw + 1; ++it) {
                const int w = it - 2;
                if (w >= 0) {
                    const int64_t slot = wave_slot(w, vv);
                    double acc = 0.0;
                    if (slot >= 0) {
                        const int vabs = (w % wpb) * V + vv;
                        const float *row_c = rows + size_t((w & 1) * V + vv) * stride + c;
                        const unsigned char *tile_lane = tiles + ((w / wpb) & 1) * tile_bytes + (c / cpb) * 32 + (vabs & 3);
                        acc = cpb == 2 ? sum_chain<2, DIM>(row_c, tile_lane, vabs >> 2, tab)
                                       : sum_chain<4, DIM>(row_c, tile_lane, vabs >> 2, tab);
                    }
                    acc = __dadd_rn(acc, __shfl_down_sync(kFullMask, acc, 1));
                    acc = __dadd_rn(acc, __shfl_down_sync(kFullMask, acc, 2));    // (c0+c1)+(c2+c3) on c = 0
                    if (c == 0 && slot >= 0)
                        p.scales[slot] = acc > 0.1 ? __fdiv_rn(norm_s[(w % 3) * V + vv], __double2float_rn(acc)) : 0.0f;
                }
                __syncwarp();
                if (it < nw && lane == 0) {
                    // stage the rows of wave `it` into the row set this warp has just finished reading
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    uint32_t bytes = 0;
                    for (int v = 0; v < V; ++v) bytes += wave_slot(it, v) >= 0 ? uint32_t(DIM * 4) : 0u;
                    if (bytes) mbar_arrive_expect_tx(&full[it & 1], bytes);
                    else mbar_arrive(&full[it & 1]);
                    for (int v = 0; v < V; ++v) {
                        const int64_t slot = wave_slot(it, v);
                        if (slot >= 0)
                            bulk_load(rows + size_t((it & 1) * V + v) * stride, p.x + (slot - slot_lo) * DIM, DIM * 4, &full[it & 1]);
                    }
                }
                __syncthreads();
            }
        } else {
            // -------------------------------------------- copy-out of finished tiles
            const int ct = tid - (V + 2) * 32;                // 0..63
            for (int it = 0; it <= nw + 1; ++it) {
                const int wf = it - 2;                        // the wave packed in the previous step
                if (wf >= 0 && wf % wpb == wpb - 1) {
                    const uint32_t *t32 = reinterpret_cast<const uint32_t *>(tiles + ((wf / wpb) & 1) * tile_bytes);
                    uint4 *dst = reinterpret_cast<uint4 *>(p.codes + size_t(first_block + wf / wpb) * tile_bytes);
#pragma unroll 4
                    for (int ch = ct; ch < ng * 2; ch += 64) {        // 16-byte chunk ch = half h of row g
                        const int g = ch >> 1, h4 = (ch & 1) * 4, s = (g >> 2) & 7;
                        const uint32_t *rowp = t32 + g * 8;
                        dst[ch] = make_uint4(rowp[(h4 + 0) ^ s], rowp[(h4 + 1) ^ s], rowp[(h4 + 2) ^ s], rowp[(h4 + 3) ^ s]);
                    }
                }
                __syncthreads();
            }
        }
    }
}

}  // namespace

bool ingest_fast_supported(int dim, int bits, bool calibrated, const void *x) {
    if (calibrated || (reinterpret_cast<uintptr_t>(x) & 15) != 0) return false;
    if (bits != 2 && bits != 3 && bits != 4) return false;
    switch (dim) {
        case 128: case 256: case 384: case 512: case 768: case 1024: case 1536: case 2048: return true;
        default: return false;
    }
}

cudaError_t launch_ingest_fast(const IngestParams &p, const float *host_boundaries, int sm_count, size_t smem_limit, uint32_t *error,
                               cudaStream_t stream) {
    if (p.n <= 0) return cudaSuccess;
    if (p.slot0 % kBlockLanes != 0) return cudaErrorInvalidValue;
    const size_t smem = fast_layout(p.dim, p.ngroups, p.bits == 2 ? 4 : 2).total;
    if (smem > smem_limit) return cudaErrorInvalidValue;
    const int64_t nblocks = (p.n + kBlockLanes - 1) / kBlockLanes;
    const unsigned grid = unsigned(std::min<int64_t>(nblocks, int64_t(sm_count)));   // one CTA per SM: it owns the register file
    Boundaries15 bnd;
    for (int i = 0; i < 15; ++i) bnd.b[i] = i < (1 << p.bits) - 1 ? host_boundaries[i] : INFINITY;
#define TV_LAUNCH_FAST(D, L2B, NB)                                                                                   \
    case D: {                                                                                                        \
        cudaError_t e = cudaFuncSetAttribute(ingest_fast_kernel<L2B, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)); \
        if (e != cudaSuccess) return e;                                                                              \
        ingest_fast_kernel<L2B, NB><<<grid, kFastThreads, smem, stream>>>(p, bnd, error);                            \
        break;                                                                                                       \
    }
    switch (p.dim) {
        TV_LAUNCH_FAST(128, 7, 1) TV_LAUNCH_FAST(256, 8, 1) TV_LAUNCH_FAST(384, 7, 3) TV_LAUNCH_FAST(512, 9, 1)
        TV_LAUNCH_FAST(768, 8, 3) TV_LAUNCH_FAST(1024, 10, 1) TV_LAUNCH_FAST(1536, 9, 3) TV_LAUNCH_FAST(2048, 11, 1)
        default: return cudaErrorInvalidValue;
    }
#undef TV_LAUNCH_FAST
    return cudaGetLastError();
}

}  // namespace tv
