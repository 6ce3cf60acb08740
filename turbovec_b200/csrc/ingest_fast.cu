// Pipelined ingest kernel for whole 32-slot code blocks (with or without a TQ+ pair): the same arithmetic as
// ingest.cu (encode::encode, turbovec/src/encode.rs:510-541 = rotate_batch_into :406-458 + encode_prerotated
// :560-652 / fused_quantize_scale_pack_scalar :1418-1476, blocked layout pack.rs:340-361), reorganised so
// that the order-fixed sequential sums no longer stall the data-parallel work.
//
// One CTA walks a contiguous range of code blocks in waves of V vectors (V = 8: three warpgroups; V = 4: two,
// for rows of which two sets of eight do not fit in shared memory) and runs its stages concurrently, one wave
// apart, with one CTA barrier per step:
//   norm warps     wave i     8 sequential f32 chains per vector straight from global memory (4 lanes per
//                             vector, two chains per lane), fixed combine tree, sqrt, reciprocal.  Two warps
//                             alternate (even and odd waves) and spread a wave over two steps: the loads come
//                             from global memory and the chains need a dozen dependent round trips.
//   staging warp   wave i     issues the bulk copies (cp.async.bulk + mbarrier transaction count) of the rows
//   V rotation     wave i-1   one warp per vector, the whole vector in registers: both rounds of permutation,
//   warps                     sign flip and Walsh-Hadamard butterflies (rotation.cuh states the order rules),
//                             Lloyd-Max quantisation through a grid table (QuantGrid), packing into the block
//                             tile, reconstruction inner product and scale
//   copy warp                 writes the finished tile of a block (ngroups x 32 bytes, word-swizzled so that the
//                             byte stores of a warp never share a bank) to the code array
// With V = 8 the two rotation warpgroups take the registers the third one gives up (setmaxnreg), so a
// 2048-coordinate vector and its permutation entries stay in registers; with V = 4 every thread may use 255.
// The row through which the two rounds exchange data uses a bank layout found by edge colouring
// (build_exchange_layout), so that neither the round-1 stores nor the round-2 gathers conflict.
//
// Reconstruction inner product.  The reference sums rotated[j] * centroid[code[j]] in f64 along four
// sequential chains (encode.rs:1418-1476) and uses the result rounded to f32, and a dependent f64 add takes
// some 45 cycles here.  The terms are the same numbers in any order (without a TQ+ pair they are even exact
// products of two f32 values), so every summation order lands within gamma * sum|terms| of their exact sum (gamma_m = m u / (1 - m u), u = 2^-53, m = additions a
// term goes through).  The rotation warp therefore sums in parallel, brackets the reference's value by
// S +- 1e-13 * A with A >= sum|products| (1e-13 > gamma_(dim/4+2) + gamma_64 for dim <= 3300), and accepts
// S when both ends of the bracket round to the same f32 and fall on the same side of the 0.1 threshold:
// rounding is monotone, so the reference's value rounds there too.  Otherwise, a few vectors in a million,
// the warp walks the four chains in the reference's order.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <vector>

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
__device__ __forceinline__ uint2 lds_u2(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ double lds_f64(uint32_t addr) {
    double v;
    asm volatile("ld.shared.f64 %0, [%1];" : "=d"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts_u8(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.u8 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ float max_nan(float a, float b) {   // NaN wins, unlike fmaxf
    float d;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
    return d;
}


// Vectors per wave = rotation warps: 8 (three warpgroups, 384 threads), or 4 (two warpgroups, 256 threads) for
// dimensions whose rows would not fit twice eight times in shared memory.  Warps V .. V+3 are the service
// warps: norm (even waves), staging, norm (odd waves), copy.
constexpr int kRotationRegs = 208, kServiceRegs = 88;   // wave of 8: 8*32*208 + 4*32*88 <= 384 * 168
constexpr int kGridCells = 1024;         // cells of the quantisation grid
constexpr float kGridTop = 8.0f * (kGridCells - 1);
constexpr float kGridMagic = 8388608.0f; // 2^23: adding it leaves the rounded integer in the low mantissa bits
constexpr double kSumBracket = 1.0e-13;  // see the head of this file

// Byte offset (cell * 8) of x in the quantisation grid.  Any monotone non-decreasing map works for the
// argument in build_quant_grid; this one costs two FMAs and a mask.
__host__ __device__ inline uint32_t grid_offset(float x, float a, float b) {
#ifdef __CUDA_ARCH__
    const float u = __saturatef(__fmaf_rn(x, a, b));
    return __float_as_uint(__fmaf_rn(u, kGridTop, kGridMagic)) & (8u * (kGridCells - 1));
#else
    float u = std::fmaf(x, a, b);
    u = u > 0.0f ? (u < 1.0f ? u : 1.0f) : 0.0f;        // NaN -> 0, like the saturating FMA
    const float v = std::fmaf(u, kGridTop, kGridMagic);
    uint32_t bits;
    std::memcpy(&bits, &v, 4);
    return bits & (8u * (kGridCells - 1));
#endif
}

struct FastLayout {
    int stride;          // floats per staged row (16-byte multiple for the bulk copies)
    size_t grid, cent, rows, tile, calib, norm, inv, bars, total;
};
__host__ __device__ inline FastLayout fast_layout(int wave, int dim, int ngroups, bool calibrated) {
    FastLayout L;
    L.stride = dim + 4;
    size_t off = 0;
    L.grid = off; off += size_t(kGridCells) * 8;       // first, so that its address is a link-time constant
    L.cent = off; off += 16 * 8;                       // centroids as f64
    L.rows = off; off += size_t(2) * wave * L.stride * 4;
    L.tile = off; off += size_t(2) * ngroups * 32;
    L.calib = off; off += calibrated ? size_t(3) * dim * 4 : 0;   // TQ+ shift, scale, 1 / scale per coordinate
    L.norm = off; off += 4 * wave * 4;
    L.inv = off; off += 4 * wave * 4;
    L.bars = off; off += 2 * 8;
    L.total = off;
    return L;
}

// Walsh-Hadamard transform of NBLK blocks of 32*R coordinates in registers, stage order len = 1, 2, 4, ...
// On entry v[b*R + r] of lane l holds coordinate l*R + r of block b: the first log2(R) stages pair registers.
// Each of the five remaining stages pairs lanes l and l ^ m.  Instead of fetching the partner's copy of every
// register, the two lanes swap one register of each pair (lane bit <-> register bit t): the lower lane ends
// up with both inputs of the pair's first register, the upper lane with both inputs of its second, each
// computes sum and difference, and the coordinate bit just processed now lives in register bit t while the
// lanes hold an already processed bit.  That halves the shuffles.  The upper lane sends its value negated, so
// that both results are single fused multiply-adds by +-1, rounded once like the add or subtract they stand
// for.  With t = stage % log2(R) the lane bits end as coordinate bits 0..4: on exit v[b*R + r] of lane l
// holds coordinate wht_row<R>(r) * 32 + l.
template <int R>
__host__ __device__ constexpr int log2_of() { int l = 0; while ((1 << l) < R) ++l; return l; }
template <int R>
__host__ __device__ constexpr int wht_row(int r) {
    constexpr int RHO = log2_of<R>();
    int bit_of[8] = {0, 1, 2, 3, 4, 5, 6, 7};         // coordinate bit held by register bit j
    for (int i = 0; i < 5; ++i) bit_of[i % RHO] = RHO + i;
    int row = 0;
    for (int j = 0; j < RHO; ++j) row |= ((r >> j) & 1) << (bit_of[j] - 5);
    return row;
}
// register k = block * R + r of a vector: its coordinates after wht_blocks are row_of(k) * 32 + lane
template <int R>
__host__ __device__ constexpr int row_of(int k) { return (k / R) * R + wht_row<R>(k % R); }
template <int R, int NBLK>
__device__ __forceinline__ void wht_blocks(float (&v)[R * NBLK], int lane) {
    constexpr int RHO = log2_of<R>();
    static_assert(RHO >= 1 && (1 << RHO) == R, "R is a power of two, at least 2");
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
#pragma unroll
    for (int i = 0; i < 5; ++i) {
        const int t = 1 << (i % RHO);
        const bool upper = (lane >> i) & 1;
        const float cs = upper ? 1.0f : -1.0f;
#pragma unroll
        for (int b = 0; b < NBLK; ++b) {
#pragma unroll
            for (int r0 = 0; r0 < R; ++r0) {
                if (r0 & t) continue;
                const int r1 = r0 | t;
                const float keep = upper ? v[b * R + r1] : v[b * R + r0];
                const float send = upper ? -v[b * R + r0] : v[b * R + r1];
                const float recv = __shfl_xor_sync(kFullMask, send, 1 << i);
                // lower lane: keep = a, recv = -b; upper lane: keep = b, recv = a
                v[b * R + r0] = __fmaf_rn(recv, cs, keep);        // a + b
                v[b * R + r1] = __fmaf_rn(keep, -cs, recv);       // a - b
            }
        }
    }
}

template <int LOG2B, int NBLK, int V, bool CALIB>
__global__ void __launch_bounds__((V + 4) * 32, 1) ingest_fast_kernel(IngestParams p, QuantGrid grid, uint32_t *error) {
    constexpr int R = 1 << (LOG2B - 5);               // registers per Hadamard block and lane
    constexpr int T = R * NBLK;                       // registers per vector and lane
    constexpr int DIM = T * 32;
    constexpr int wpb = kBlockLanes / V;
    constexpr int kFastThreads = (V + 4) * 32;
    static_assert(V == 8 || V == 4, "waves of 8 or 4 vectors");
    static_assert(T % 4 == 0, "the packing below handles whole groups of four registers");
    constexpr int kNormBatch = (DIM / 16) % 16 == 0 ? 16 : 8;   // chain steps per load batch; a half wave has DIM / 16 steps
    extern __shared__ __align__(128) unsigned char smem[];
    const int ng = p.ngroups;
    const int cpb = p.bits == 2 ? 4 : 2;              // codes per byte (3-bit codes sit in 4-bit fields)
    const FastLayout L = fast_layout(V, DIM, ng, CALIB);
    float *rows = reinterpret_cast<float *>(smem + L.rows);
    unsigned char *tiles = smem + L.tile;
    float *norm_s = reinterpret_cast<float *>(smem + L.norm);     // [4][8]
    float *inv_s = reinterpret_cast<float *>(smem + L.inv);       // [4][8]
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
    for (int i = tid; i < kGridCells; i += kFastThreads) reinterpret_cast<uint2 *>(smem + L.grid)[i] = grid.cells[i];
    if (tid < 16) reinterpret_cast<double *>(smem + L.cent)[tid] = double(p.centroids[tid]);   // the array has 16 slots
    if constexpr (CALIB) {
        float *cal = reinterpret_cast<float *>(smem + L.calib);
        for (int i = tid; i < DIM; i += kFastThreads) {
            cal[i] = p.shift[i]; cal[DIM + i] = p.scale_tq[i]; cal[2 * DIM + i] = p.inv_scale_tq[i];
        }
    }
    __syncthreads();

    // slot of vector `v` of wave `w`, or -1 past the new rows (padding lanes of the last block)
    auto wave_slot = [&](int w, int v) -> int64_t {
        const int64_t s = (first_block + w / wpb) * 32 + (w % wpb) * V + v;
        return s < slot_hi ? s : -1;
    };

    if (warp < V) {
        if constexpr (V == 8) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRotationRegs) : "memory");
        // ------------------------------------------------ rotation + quantisation: one vector per warp
        uint32_t pk[T];          // per register: round-1 byte offset | sign << 15, round-2 the same in the high half
#pragma unroll
        for (int k = 0; k < T; ++k) {
            const int dst = (k / R) * (32 * R) + lane * R + (k % R);       // coordinate this register gathers (see wht_blocks)
            const uint32_t e0 = p.perm0[dst], e1 = (p.perm1_exchange ? p.perm1_exchange : p.perm1)[dst];
            pk[k] = ((e0 & 0x7fffu) << 2) | (e0 & 0x8000u) | ((((e1 & 0x7fffu) << 2) | (e1 & 0x8000u)) << 16);
        }
        // byte offset of each register's place within its row of the exchange layout, four per word
        // (lane * 4 for plain rows); not kept for the largest vectors, which have no registers to spare
        constexpr bool kExchange = T <= 48;
        uint32_t sbank[kExchange ? T / 4 : 1];
        if constexpr (kExchange) {
#pragma unroll
            for (int j = 0; j < T / 4; ++j) {
                uint32_t wd = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    wd |= (p.store_bank ? uint32_t(p.store_bank[(4 * j + i) * 32 + lane]) : uint32_t(lane * 4)) << (8 * i);
                sbank[j] = wd;
            }
        }
        const float isb = p.inv_sqrt_block;
        const float ga = grid.a, gb = grid.b;
        const uint32_t grid_base = smem_u32(smem + L.grid), cent_base = smem_u32(smem + L.cent);
        const uint32_t cal_lane = smem_u32(smem + L.calib) + lane * 4;   // TQ+ tables at this lane's coordinates
        float cmax = 0.0f;                            // largest |centroid|
        for (int i = 0; i < (1 << p.bits); ++i) cmax = fmaxf(cmax, fabsf(p.centroids[i]));
        const int q = lane & (cpb - 1);               // this lane packs the registers k = q (mod cpb)

        for (int it = 0; it <= nw + 1; ++it) {
            const int w = it - 1;
            if (w >= 0 && w < nw) {
                const int64_t slot = wave_slot(w, warp);
                uint32_t cw[(T + 7) / 8];             // 4-bit code of coordinates kk*32 + lane in nibble kk % 8 of word kk / 8
#pragma unroll
                for (int i = 0; i < (T + 7) / 8; ++i) cw[i] = 0;
                float *row = rows + size_t((w & 1) * V + warp) * stride;
                if (slot >= 0 && mbar_wait(&full[w & 1], (w >> 1) & 1, error)) {
                    const uint32_t rb = smem_u32(row), rl = rb + lane * 4;
                    const float inv = inv_s[(w & 3) * V + warp];
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
                    wht_blocks<R, NBLK>(v, lane);
#pragma unroll
                    for (int k = 0; k < T; ++k) {
                        uint32_t at = rl;
                        if constexpr (kExchange) at = rb + __byte_perm(sbank[k >> 2], 0, 0x4440 + (k & 3));
                        sts_f32(at + row_of<R>(k) * 128, __fmul_rn(v[k], isb));
                    }
                    __syncwarp();
                    // round 2
#pragma unroll
                    for (int k = 0; k < T; ++k) {
                        const float x = lds_f32(rb + ((pk[k] >> 16) & 0x7ffcu));
                        v[k] = __uint_as_float(__float_as_uint(x) ^ (pk[k] & 0x80000000u));
                    }
                    __syncwarp();
                    wht_blocks<R, NBLK>(v, lane);
                    double sacc[8];                                   // independent partial sums hide the f64 latency
#pragma unroll
                    for (int i = 0; i < 8; ++i) sacc[i] = 0.0;
                    float aacc = 0.0f;                                // sum |y| of this lane (uncalibrated)
                    double tabs = 0.0;                                // sum |term| of this lane (calibrated)
#pragma unroll
                    for (int k = 0; k < T; ++k) {
                        const float y = __fmul_rn(v[k], isb);
                        v[k] = y;
                        const int kk = row_of<R>(k);               // this register holds coordinate kk * 32 + lane
                        float c = y, sh = 0.0f;
                        if constexpr (CALIB) {                     // (rot + shift) * scale, encode.rs:1447
                            sh = lds_f32(cal_lane + kk * 128);
                            c = __fmul_rn(__fadd_rn(y, sh), lds_f32(cal_lane + DIM * 4 + kk * 128));
                        }
                        // code = number of boundaries strictly below c (encode.rs:1447-1451): the cell of c
                        // knows how many lie in lower cells and the one boundary, if any, inside the cell
                        const uint2 cell = lds_u2(grid_base + grid_offset(c, ga, gb));
                        const uint32_t code8 = cell.y + (c > __uint_as_float(cell.x) ? 8u : 0u);   // 8 * code
                        cw[kk >> 3] += (kk & 7) == 0 ? code8 >> 3 : code8 * (1u << (4 * (kk & 7) - 3));
                        if constexpr (CALIB) {
                            // rot * (centroid / scale - shift) in f64, every operation rounded as in encode.rs:276-278, 1455
                            const double recon = __dsub_rn(__dmul_rn(lds_f64(cent_base + code8), double(lds_f32(cal_lane + 2 * DIM * 4 + kk * 128))), double(sh));
                            const double term = __dmul_rn(double(y), recon);
                            sacc[k & 7] = __dadd_rn(sacc[k & 7], term);
                            tabs = __dadd_rn(tabs, fabs(term));
                        } else {
                            sacc[k & 7] = __fma_rn(double(y), lds_f64(cent_base + code8), sacc[k & 7]);
                            aacc += fabsf(y);
                        }
                    }
                    double S = ((sacc[0] + sacc[1]) + (sacc[2] + sacc[3])) + ((sacc[4] + sacc[5]) + (sacc[6] + sacc[7]));
#pragma unroll
                    for (int m = 1; m < 32; m <<= 1) {
                        S += __shfl_xor_sync(kFullMask, S, m);        // commutative: every lane ends with the same bits
                        if constexpr (CALIB) tabs += __shfl_xor_sync(kFullMask, tabs, m);
                        else aacc += __shfl_xor_sync(kFullMask, aacc, m);
                    }
                    // A >= sum |terms|.  Uncalibrated: sum |y| * max|centroid| (the factor covers the f32 rounding of
                    // aacc).  Calibrated: the terms are rounded values, the same in any order, and their absolute
                    // sum in f64 is off by far less than the factor.
                    const double A = CALIB ? tabs * 1.000001 : double(aacc) * double(cmax) * 1.0001;
                    const double lo = S - kSumBracket * A, hi = S + kSumBracket * A;
                    const float flo = __double2float_rn(lo), fhi = __double2float_rn(hi);
                    const bool certain = flo == fhi && (lo > 0.1) == (hi > 0.1) && p.exact_sums == 0;
                    float inner_f = flo;
                    bool above = lo > 0.1;
                    if (!certain) {
                        // the reference's own order: chain c over j = c (mod 4) ascending, (c0+c1)+(c2+c3)
#pragma unroll
                        for (int k = 0; k < T; ++k) sts_f32(rl + row_of<R>(k) * 128, v[k]);
                        __syncwarp();
                        double acc = 0.0;
                        if (lane < 4) {
                            const float *cal = reinterpret_cast<const float *>(smem + L.calib);
                            for (int j = lane; j < DIM; j += 4) {
                                const float y = row[j];
                                float c = y, sh = 0.0f;
                                if constexpr (CALIB) { sh = cal[j]; c = __fmul_rn(__fadd_rn(y, sh), cal[DIM + j]); }
                                const uint2 cell = lds_u2(grid_base + grid_offset(c, ga, gb));
                                const uint32_t code8 = cell.y + (c > __uint_as_float(cell.x) ? 8u : 0u);
                                if constexpr (CALIB) {
                                    const double recon = __dsub_rn(__dmul_rn(lds_f64(cent_base + code8), double(cal[2 * DIM + j])), double(sh));
                                    acc = __dadd_rn(acc, __dmul_rn(double(y), recon));
                                } else {
                                    acc = __fma_rn(double(y), lds_f64(cent_base + code8), acc);   // exact product: one rounding
                                }
                            }
                        }
                        acc = __dadd_rn(acc, __shfl_down_sync(kFullMask, acc, 1));
                        acc = __dadd_rn(acc, __shfl_down_sync(kFullMask, acc, 2));
                        acc = __shfl_sync(kFullMask, acc, 0);
                        inner_f = __double2float_rn(acc);
                        above = acc > 0.1;
                        __syncwarp();
                    }
                    if (lane == 0) p.scales[slot] = above ? __fdiv_rn(norm_s[(w & 3) * V + warp], inner_f) : 0.0f;
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
        if constexpr (V == 8) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kServiceRegs) : "memory");
        if (warp == V || warp == V + 2) {
            // -------------------------------------------- norms: this warp takes the waves of one parity and
            // spreads each over two steps (first half of the chains in step w - 1, second half in step w)
            const int parity = warp == V ? 0 : 1;
            const int vv = lane >> 2, pp = lane & 3;
            float a0 = 0.0f, a1 = 0.0f;
            for (int it = 0; it <= nw + 1; ++it) {
                const bool second = (it & 1) == parity;               // else: first half of wave it + 1
                const int w = second ? it : it + 1;
                if (w < nw) {
                    if (!second && w + 2 < nw && lane < V) {
                        // pull this warp's next wave into L2
                        const int64_t slot = wave_slot(w + 2, lane);
                        if (slot >= 0)
                            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.x + (slot - slot_lo) * DIM), "r"(DIM * 4) : "memory");
                    }
                    const int64_t slot = vv < V ? wave_slot(w, vv) : -1;
                    // chains 2pp and 2pp+1: x[j]^2 summed over j = chain (mod 8) in ascending j (encode.rs:900-932)
                    const bool whole = second && it == 0;             // wave 0 has no earlier step
                    if (!second || whole) { a0 = 0.0f; a1 = 0.0f; }
                    if (slot >= 0) {
                        const float2 *src = reinterpret_cast<const float2 *>(p.x + (slot - slot_lo) * DIM + 2 * pp);
                        const int t_begin = second && !whole ? DIM / 16 : 0, t_end = second ? DIM / 8 : DIM / 16;
#pragma unroll 1
                        for (int t0 = t_begin; t0 < t_end; t0 += kNormBatch) {
                            float2 x[kNormBatch];                     // loads in flight per lane
#pragma unroll
                            for (int u = 0; u < kNormBatch; ++u) x[u] = __ldg(src + 4 * (t0 + u));
#pragma unroll
                            for (int u = 0; u < kNormBatch; ++u) {
                                a0 = __fadd_rn(a0, __fmul_rn(x[u].x, x[u].x));
                                a1 = __fadd_rn(a1, __fmul_rn(x[u].y, x[u].y));
                            }
                        }
                    }
                    if (second) {
                        float s = __fadd_rn(a0, a1);                              // (c0+c1), (c2+c3), (c4+c5), (c6+c7)
                        s = __fadd_rn(s, __shfl_down_sync(kFullMask, s, 1));      // valid on pp = 0 and pp = 2
                        s = __fadd_rn(s, __shfl_down_sync(kFullMask, s, 2));      // valid on pp = 0
                        if (pp == 0 && vv < V) {
                            const float nv = __fsqrt_rn(s);
                            norm_s[(w & 3) * V + vv] = nv;
                            inv_s[(w & 3) * V + vv] = nv > kMinNorm ? __fdiv_rn(1.0f, nv) : 0.0f;    // encode.rs:446
                        }
                    }
                }
                __syncthreads();
            }
        } else if (warp == V + 1) {
            // -------------------------------------------- row staging: wave `it` lands while wave it - 1 rotates;
            // its row set was last read by the rotation of wave it - 2, one barrier ago
            for (int it = 0; it <= nw + 1; ++it) {
                if (it < nw) {
                    const int64_t slot = lane < V ? wave_slot(it, lane) : -1;
                    const uint32_t live = __ballot_sync(kFullMask, slot >= 0);
                    if (lane == 0) {
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        if (live) mbar_arrive_expect_tx(&full[it & 1], uint32_t(__popc(live)) * uint32_t(DIM * 4));
                        else mbar_arrive(&full[it & 1]);
                    }
                    __syncwarp();
                    if (slot >= 0)
                        bulk_load(rows + size_t((it & 1) * V + lane) * stride, p.x + (slot - slot_lo) * DIM, DIM * 4, &full[it & 1]);
                }
                __syncthreads();
            }
        } else {
            // -------------------------------------------- copy-out of finished tiles
            for (int it = 0; it <= nw + 1; ++it) {
                const int wf = it - 2;                        // the wave packed in the previous step
                if (wf >= 0 && wf % wpb == wpb - 1) {
                    const uint32_t *t32 = reinterpret_cast<const uint32_t *>(tiles + ((wf / wpb) & 1) * tile_bytes);
                    uint4 *dst = reinterpret_cast<uint4 *>(p.codes + size_t(first_block + wf / wpb) * tile_bytes);
#pragma unroll 4
                    for (int ch = lane; ch < ng * 2; ch += 32) {      // 16-byte chunk ch = half h of row g
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

// For every boundary: the grid cell it falls in.  grid_offset is monotone non-decreasing in x, so for a
// value x in cell c every boundary in a lower cell is below x and every boundary in a higher cell is not;
// only a boundary in cell c itself needs the exact comparison.  The table is valid when no two boundaries
// share a cell; then code(x) = lower[c] + (x > inside[c]).
bool build_quant_grid(const float *boundaries, int count, QuantGridHost &out) {
    if (count < 1 || count > 15) return false;
    for (int i = 0; i + 1 < count; ++i)
        if (!(boundaries[i] < boundaries[i + 1])) return false;
    const float lo = boundaries[0], hi = boundaries[count - 1];
    const float pad = count > 1 ? (hi - lo) / 64.0f : 1.0f;
    const float span = (hi - lo) + 2.0f * pad;
    if (!(span > 0.0f) || !std::isfinite(span)) return false;
    out.a = 1.0f / span;
    out.b = -(lo - pad) / span;
    std::vector<int> cell_of(count);
    for (int i = 0; i < count; ++i) {
        cell_of[i] = int(grid_offset(boundaries[i], out.a, out.b) / 8);
        if (i > 0 && cell_of[i] == cell_of[i - 1]) return false;
    }
    out.cells.assign(kGridCells, QuantCell{});
    int below = 0;       // boundaries in cells lower than c
    for (int c = 0, i = 0; c < kGridCells; ++c) {
        float inside = std::numeric_limits<float>::max();     // finite inputs never exceed it
        if (i < count && cell_of[i] == c) inside = boundaries[i];
        std::memcpy(&out.cells[c].boundary_bits, &inside, 4);
        out.cells[c].code8 = uint32_t(below) * 8u;
        if (i < count && cell_of[i] == c) { ++i; ++below; }
    }
    return true;
}

// Edge colouring of a bipartite multigraph in which every vertex has degree `colours`: colour[e] in
// [0, colours) such that no two edges at a vertex share a colour (Koenig).  Alternating-path algorithm.
static void colour_edges(int n_left, int n_right, int colours, const std::vector<int> &left, const std::vector<int> &right,
                         std::vector<int> &colour) {
    const int m = int(left.size());
    colour.assign(m, -1);
    std::vector<int> at_l(size_t(n_left) * colours, -1), at_r(size_t(n_right) * colours, -1);   // edge with colour c at a vertex
    for (int e = 0; e < m; ++e) {
        const int u = left[e], v = right[e];
        int a = 0, b = 0;
        while (at_l[size_t(u) * colours + a] >= 0) ++a;      // free at u
        while (at_r[size_t(v) * colours + b] >= 0) ++b;      // free at v
        if (a != b) {
            // colour a is taken at v: walk the a/b alternating path that starts at v and swap its colours;
            // it cannot come back to u, where a is free
            std::vector<int> path;
            int x = v, want = a;
            bool on_right = true;
            for (;;) {
                const int f = on_right ? at_r[size_t(x) * colours + want] : at_l[size_t(x) * colours + want];
                if (f < 0) break;
                path.push_back(f);
                x = on_right ? left[f] : right[f];
                on_right = !on_right;
                want = want == a ? b : a;
            }
            for (int f : path) {
                const int c = colour[f];
                at_l[size_t(left[f]) * colours + c] = -1;
                at_r[size_t(right[f]) * colours + c] = -1;
            }
            for (int f : path) {
                const int c = colour[f] == a ? b : a;
                colour[f] = c;
                at_l[size_t(left[f]) * colours + c] = f;
                at_r[size_t(right[f]) * colours + c] = f;
            }
        }
        colour[e] = a;
        at_l[size_t(u) * colours + a] = e;
        at_r[size_t(v) * colours + a] = e;
    }
}

static int wht_row_rt(int R, int r) {
    int rho = 0;
    while ((1 << rho) < R) ++rho;
    int bit_of[8] = {0, 1, 2, 3, 4, 5, 6, 7};
    for (int i = 0; i < 5; ++i) bit_of[i % rho] = rho + i;
    int row = 0;
    for (int j = 0; j < rho; ++j) row |= ((r >> j) & 1) << (bit_of[j] - 5);
    return row;
}

// Layout of the row through which the two rotation rounds exchange data.  Store instruction k of the warp
// writes the 32 coordinates row_of(k)*32 + lane, gather instruction k' of round 2 reads the 32 coordinates
// perm1[dst(k', lane)]; each coordinate is an edge between its store and its gather instruction, and a
// 32-colouring of the edges gives every coordinate a bank such that neither kind of instruction has two lanes
// on one bank.  Coordinate e then lives in word (e / 32) * 32 + bank(e): still in the 128-byte row of its
// store instruction, at another place.
bool build_exchange_layout(int dim, const uint16_t *perm1_packed, ExchangeLayoutHost &out) {
    const int block = dim & -dim;
    const int R = block / 32, T = dim / 32;
    if (R < 2 || dim % 32 != 0 || dim > 8192) return false;
    std::vector<int> store_of(dim), gather_of(dim, -1), lane_of_store(dim), row_of_store(dim);
    for (int k = 0; k < T; ++k)
        for (int l = 0; l < 32; ++l) {
            const int e = ((k / R) * R + wht_row_rt(R, k % R)) * 32 + l;
            store_of[e] = k;
            lane_of_store[e] = l;
            row_of_store[e] = e / 32;
            const int dst = (k / R) * (32 * R) + l * R + (k % R);
            const int src = perm1_packed[dst] & 0x7fff;
            if (src >= dim || gather_of[src] >= 0) return false;
            gather_of[src] = k;
        }
    std::vector<int> colour;
    colour_edges(T, T, 32, store_of, gather_of, colour);
    out.T = T;
    out.store_bank.assign(dim, 0);
    out.perm1_exchange.assign(dim, 0);
    for (int e = 0; e < dim; ++e) out.store_bank[store_of[e] * 32 + lane_of_store[e]] = uint8_t(colour[e] * 4);   // byte offset in the row
    for (int dst = 0; dst < dim; ++dst) {
        const int src = perm1_packed[dst] & 0x7fff;
        out.perm1_exchange[dst] = uint16_t((row_of_store[src] * 32 + colour[src]) | (perm1_packed[dst] & 0x8000));
    }
    return true;
}

// Worst number of lanes of one instruction on one bank: (stores, gathers) of the layout, and of the
// linear layout for comparison.  1 = conflict-free.
void exchange_layout_conflicts(int dim, const uint16_t *perm1_packed, const ExchangeLayoutHost *layout, int *store_max, int *gather_max) {
    const int block = dim & -dim, R = block / 32, T = dim / 32;
    *store_max = *gather_max = 0;
    for (int k = 0; k < T; ++k) {
        int sb[32] = {0}, gb[32] = {0};
        for (int l = 0; l < 32; ++l) {
            const int dst = (k / R) * (32 * R) + l * R + (k % R);
            int s_bank, g_bank;
            if (layout) { s_bank = layout->store_bank[k * 32 + l] / 4; g_bank = (layout->perm1_exchange[dst] & 0x7fff) % 32; }
            else { s_bank = l; g_bank = (perm1_packed[dst] & 0x7fff) % 32; }
            *store_max = std::max(*store_max, ++sb[s_bank]);
            *gather_max = std::max(*gather_max, ++gb[g_bank]);
        }
    }
}

// Host evaluation of a grid, the same lookup the kernel performs.
uint32_t quant_grid_code(const QuantGridHost &g, float x) {
    const QuantCell &c = g.cells[grid_offset(x, g.a, g.b) / 8];
    float inside;
    std::memcpy(&inside, &c.boundary_bits, 4);
    return c.code8 / 8 + (x > inside ? 1u : 0u);
}

namespace {
// 8 vectors per wave where two row sets of 8 fit into shared memory next to the tiles, else 4
int wave_for(int dim, int ngroups, bool calibrated, size_t smem_limit) {
    if (dim <= 2048 && fast_layout(8, dim, ngroups, calibrated).total <= smem_limit) return 8;
    return fast_layout(4, dim, ngroups, calibrated).total <= smem_limit ? 4 : 0;
}
}  // namespace

bool ingest_fast_supported(int dim, int bits, int ngroups, bool calibrated, const void *x, size_t smem_limit) {
    if ((reinterpret_cast<uintptr_t>(x) & 15) != 0) return false;
    if (bits != 2 && bits != 3 && bits != 4) return false;
    switch (dim) {
        case 128: case 256: case 384: case 512: case 768: case 1024: case 1536: case 2048: case 3072: break;
        default: return false;
    }
    return wave_for(dim, ngroups, calibrated, smem_limit) != 0;
}

cudaError_t launch_ingest_fast(const IngestParams &p, const QuantGrid &grid, int sm_count, size_t smem_limit, uint32_t *error,
                               cudaStream_t stream) {
    if (p.n <= 0) return cudaSuccess;
    if (p.slot0 % kBlockLanes != 0 || grid.cells == nullptr) return cudaErrorInvalidValue;
    const bool calibrated = p.shift != nullptr;
    const int wave = wave_for(p.dim, p.ngroups, calibrated, smem_limit);
    if (wave == 0) return cudaErrorInvalidValue;
    const size_t smem = fast_layout(wave, p.dim, p.ngroups, calibrated).total;
    const int64_t nblocks = (p.n + kBlockLanes - 1) / kBlockLanes;
    const unsigned nctas = unsigned(std::min<int64_t>(nblocks, int64_t(sm_count)));   // one CTA per SM: it owns the register file
#define TV_LAUNCH_FAST_VC(L2B, NB, VV, CC)                                                                           \
    {                                                                                                                \
        cudaError_t e = cudaFuncSetAttribute(ingest_fast_kernel<L2B, NB, VV, CC>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)); \
        if (e != cudaSuccess) return e;                                                                              \
        ingest_fast_kernel<L2B, NB, VV, CC><<<nctas, (VV + 4) * 32, smem, stream>>>(p, grid, error);                 \
    }
#define TV_LAUNCH_FAST_V(L2B, NB, VV)                                                                                \
    {                                                                                                                \
        if (calibrated) TV_LAUNCH_FAST_VC(L2B, NB, VV, true) else TV_LAUNCH_FAST_VC(L2B, NB, VV, false)              \
    }
#define TV_LAUNCH_FAST(D, L2B, NB)                                                                                   \
    case D:                                                                                                          \
        if (wave == 8) TV_LAUNCH_FAST_V(L2B, NB, 8) else TV_LAUNCH_FAST_V(L2B, NB, 4)                                \
        break;
    switch (p.dim) {
        TV_LAUNCH_FAST(128, 7, 1) TV_LAUNCH_FAST(256, 8, 1) TV_LAUNCH_FAST(384, 7, 3) TV_LAUNCH_FAST(512, 9, 1)
        TV_LAUNCH_FAST(768, 8, 3) TV_LAUNCH_FAST(1024, 10, 1) TV_LAUNCH_FAST(1536, 9, 3)
        case 2048:
            if (wave == 8) TV_LAUNCH_FAST_V(11, 1, 8) else TV_LAUNCH_FAST_V(11, 1, 4)
            break;
        case 3072: TV_LAUNCH_FAST_V(10, 3, 4) break;
        default: return cudaErrorInvalidValue;
    }
#undef TV_LAUNCH_FAST
#undef TV_LAUNCH_FAST_V
#undef TV_LAUNCH_FAST_VC
    return cudaGetLastError();
}

}  // namespace tv
