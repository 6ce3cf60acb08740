// Search-side kernels: query preparation, allow-mask utilities, the block scans and top-k selection.
//
// Reference path restated: search::search (turbovec/src/search.rs:3206-4353):
//   rotate queries (:3237-3242) -> TQ+ inverse (:3154-3186) -> per-query tables (:2856-2994, :2806-2846)
//   -> block scan with whole-block mask skip (:3015-3029) and per-vector scale -> top-k under the order
//   (score desc, slot asc) (:236-252, :4285-4298).
// Integer sums are exact here as they are in every reference kernel; the float epilogue reproduces the
// reference's rounding sequence for the selected score mode.
#include <algorithm>

#include "search.cuh"

#include <cfloat>

#include "rotation.cuh"
#include "scan_common.cuh"

namespace tv {
namespace {

// =====================================================================================================
// Query preparation: one CTA per query.
// =====================================================================================================
__device__ __forceinline__ float block_max(float v, float *red, int tid, int nthreads) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFullMask, v, o));
    if ((tid & 31) == 0) red[tid >> 5] = v;
    __syncthreads();
    float r = red[0];
    for (int w = 1; w < (nthreads >> 5); ++w) r = fmaxf(r, red[w]);
    __syncthreads();
    return r;
}

__device__ __forceinline__ int8_t round_clamp_i8(float v) {
    float r = roundf(v);                       // half away from zero, as Rust's f32::round
    r = fminf(fmaxf(r, -127.0f), 127.0f);
    return int8_t(int(r));
}

template <int LOG2B>
__global__ void __launch_bounds__(128) query_prep_kernel(QueryPrepParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int dim = p.dim, ng = p.ngroups, stride = dim + 8;
    float *rowA = reinterpret_cast<float *>(smem_raw);
    float *rowB = rowA + stride;
    uint16_t *perm0 = reinterpret_cast<uint16_t *>(rowB + stride);
    uint16_t *perm1 = perm0 + dim;
    float *mins = reinterpret_cast<float *>(perm0);     // reused after the rotation: 2*ng floats <= 4*dim bytes
    __shared__ float red[4];
    __shared__ float s_scalar[2];

    const int q = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float *src = p.queries + size_t(q) * dim;
    for (int i = tid; i < dim; i += blockDim.x) {
        const float v = src[i];
        rowA[i] = v;
        if (!(fabsf(v) < 1e16f)) atomicMin(p.first_invalid, (unsigned long long)(size_t(q) * dim + i));
        perm0[i] = p.perm0[i];
        perm1[i] = p.perm1[i];
    }
    __syncthreads();
    if (warp == 0)   // Rotation::apply: no normalisation (search.rs:3237-3242)
        rotate_row<LOG2B>(rowA, rowB, perm0, perm1, dim, p.inv_sqrt_block, false, 1.0f, lane);
    __syncthreads();

    // TQ+ inverse (search.rs:3154-3186): q[d] / scale[d]; bias correction = -(sum q[d]*shift[d]) in f64,
    // accumulated sequentially in d.
    float bias_corr = 0.0f;
    if (p.shift != nullptr) {
        if (tid == 0) {
            double bc = 0.0;
            for (int d = 0; d < dim; ++d) bc = __dsub_rn(bc, __dmul_rn(double(rowA[d]), double(p.shift[d])));
            s_scalar[0] = __double2float_rn(bc);
        }
        __syncthreads();
        bias_corr = s_scalar[0];
        for (int d = tid; d < dim; d += blockDim.x) rowA[d] = __fdiv_rn(rowA[d], p.scale_tq[d]);
        __syncthreads();
    }
    for (int d = tid; d < dim; d += blockDim.x) p.q_rot[size_t(q) * dim + d] = rowA[d];

    if (p.mode == kModePermuteDot) {
        // search.rs:2806-2846: one scale for the row, weights = clamp(round(q * (1/qs)), +-127)
        float m = 0.0f;
        for (int d = tid; d < dim; d += blockDim.x) m = fmaxf(m, fabsf(rowA[d]));
        const float qmax = block_max(m, red, tid, blockDim.x);
        float qs = __fdiv_rn(qmax, 127.0f), inv_qs;
        if (qs >= FLT_MIN) inv_qs = __fdiv_rn(1.0f, qs);
        else { qs = 1.0f; inv_qs = 1.0f; }
        if (tid == 0) {
            p.qscale[q] = __fmul_rn(p.level_scale, qs);
            p.qbias[q] = __fadd_rn(0.0f, bias_corr);
        }
        int8_t *wrow = p.weights + size_t(q) * p.dim_pad;
        for (int d = tid; d < dim; d += blockDim.x) wrow[d ^ 1] = round_clamp_i8(__fmul_rn(rowA[d], inv_qs));
        // mma.sync A fragments.  k-step ks covers byte-groups 16ks..16ks+15; thread t of a quad owns
        // groups 16ks + t + {0,4,8,12}; register byte order follows the nibble order of a code byte
        // (low nibble = odd coordinate 2g+1, high nibble = even coordinate 2g; search.rs:2787-2790).
        const int ksteps = (ng + 15) / 16;
        const int m_tile = q >> 4, rr = q & 15, r = rr & 7, hi_row = rr >> 3;
        for (int idx = tid; idx < ksteps * 8; idx += blockDim.x) {
            const int ks = idx >> 3, t = (idx >> 1) & 3, half = idx & 1;
            const int ga = 16 * ks + t + 8 * half, gb = ga + 4;
            uint32_t word = 0;
            const int dims[4] = {2 * ga + 1, 2 * ga, 2 * gb + 1, 2 * gb};
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                int8_t w = 0;
                if (dims[b] < dim) w = round_clamp_i8(__fmul_rn(rowA[dims[b]], inv_qs));
                word |= uint32_t(uint8_t(w)) << (8 * b);
            }
            const size_t frag = ((size_t(ks) * p.mtiles_total + m_tile) * 32 + (r * 4 + t)) * 4 + (half * 2 + hi_row);
            p.wfrag[frag] = word;
        }
    } else {
        // search.rs:2856-2994.  Entry = sum over the nibble's coordinates of q[d]*centroid[code]
        // (f32, coordinate order, separately rounded multiply and add).
        const int cpb = 8 / p.bits, cpn = cpb / 2;
        const unsigned code_mask = (1u << p.bits) - 1u;
        auto entry = [&](int d0, unsigned nib) {
            float s = 0.0f;
            for (int c = 0; c < cpn; ++c) {
                const unsigned code = (nib >> ((cpn - 1 - c) * p.bits)) & code_mask;
                s = __fadd_rn(s, __fmul_rn(rowA[d0 + c], p.centroids[code]));
            }
            return s;
        };
        float span = 0.0f;
        for (int h = tid; h < 2 * ng; h += blockDim.x) {           // h = 2*g + half
            const int d0 = (h >> 1) * cpb + (h & 1) * cpn;
            float mn = FLT_MAX, mx = -FLT_MAX;
            for (unsigned nib = 0; nib < 16; ++nib) {
                const float s = entry(d0, nib);
                if (s < mn) mn = s;
                if (s > mx) mx = s;
            }
            mins[h] = mn;
            span = fmaxf(span, __fsub_rn(mx, mn));
        }
        const float max_span = block_max(span, red, tid, blockDim.x);
        float scale = max_span > 0.0f ? __fdiv_rn(max_span, 127.0f) : 1.0f;
        float inv_scale;
        if (scale >= FLT_MIN) inv_scale = __fdiv_rn(1.0f, scale);
        else { scale = 1.0f; inv_scale = 1.0f; }
        if (tid == 0) {
            float bias = 0.0f;                                      // sequential in g (search.rs:2910)
            for (int g = 0; g < ng; ++g) bias = __fadd_rn(bias, __fadd_rn(mins[2 * g], mins[2 * g + 1]));
            p.qscale[q] = scale;
            p.qbias[q] = __fadd_rn(bias, bias_corr);                // search.rs:3260
        }
        uint8_t *lut = p.luts + size_t(q) * p.lut_pitch;
        for (int e = tid; e < ng * 32; e += blockDim.x) {
            const int h = e >> 4;
            const unsigned nib = e & 15;
            const int d0 = (h >> 1) * cpb + (h & 1) * cpn;
            float r = roundf(__fmul_rn(__fsub_rn(entry(d0, nib), mins[h]), inv_scale));
            r = fminf(fmaxf(r, 0.0f), 127.0f);
            lut[e] = uint8_t(int(r));
        }
    }
}

// =====================================================================================================
// Allow-mask utilities
// =====================================================================================================
__global__ void pack_bool_mask_kernel(const uint8_t *mask_bool, int64_t n, uint32_t *words32) {
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const bool on = i < n && mask_bool[i] != 0;
    const unsigned w = __ballot_sync(kFullMask, on);
    if ((threadIdx.x & 31) == 0 && (i >> 5) < ((n + 63) / 64) * 2) words32[i >> 5] = w;
}

__global__ void scatter_slots_kernel(const uint32_t *slots, int64_t count, uint32_t *words32) {
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) atomicOr(&words32[slots[i] >> 5], 1u << (slots[i] & 31));
}

__global__ void mask_stats_kernel(uint32_t *words32, int64_t n, unsigned long long *n_allowed, uint32_t *live_blocks,
                                  uint32_t *n_live) {
    const int64_t nblocks = (n + 31) / 32;
    const int64_t b = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    unsigned w = 0;
    if (b < nblocks) {
        w = words32[b];
        const int64_t rem = n - b * 32;
        if (rem < 32) { w &= (1u << rem) - 1u; words32[b] = w; }
    }
    // ordered-within-warp append keeps neighbouring live blocks adjacent in the list
    const unsigned live = __ballot_sync(kFullMask, w != 0);
    unsigned cnt = __popc(w);
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(kFullMask, cnt, o);
    const int lane = threadIdx.x & 31;
    unsigned base = 0;
    if (lane == 0 && live) {
        base = atomicAdd(n_live, __popc(live));
        atomicAdd(n_allowed, (unsigned long long)cnt);
    }
    base = __shfl_sync(kFullMask, base, 0);
    if (w != 0) live_blocks[base + __popc(live & ((1u << lane) - 1u))] = uint32_t(b);
}

// =====================================================================================================
// Permute-dot scan (4-bit codes): S[q][v] = sum_d W[q][d] * level[code[v][d]], exact in int32
// (search.rs:1392-1543), then fma((f32)S, scale_q, bias_q) * vec_scale[v] (search.rs:1523, 1793).
//
// CTA = 8 consumer warps + 1 producer warp.  A tile is 8 code blocks (256 vectors), one per consumer
// warp.  The producer streams the tile's codes in chunks of kChunkRows byte-group rows per block with
// bulk asynchronous copies into a ring of kStages shared-memory stages (full/empty mbarriers).  A
// consumer turns 16 rows x 4 bytes into the B fragments of four m16n8k32 MMAs: the byte of vector
// 4i+j in row g sits in byte j of the 32-bit word at (g, quad i), so one word feeds the four n-tiles
// j = 0..3 of quad i; nibbles become int8 levels with three byte-permutes per four codes.
// =====================================================================================================
constexpr int kConsumerWarps = 8;
constexpr int kChunkRows = 64;                                // byte-group rows per block per stage
constexpr int kStageBytes = kConsumerWarps * kChunkRows * kLanes;
constexpr int kStages = 4;

template <int MT, bool SPLIT>
__global__ void __launch_bounds__((kConsumerWarps + 1) * 32, MT == 1 ? (SPLIT ? 2 : 3) : (MT == 2 ? 2 : 1))
scan_pd_kernel(ScanParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    uint8_t *stage_mem = smem_raw;
    __shared__ uint64_t full_bar[kStages], empty_bar[kStages];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ng = p.ngroups;
    const int n_chunks = (ng + kChunkRows - 1) / kChunkRows;
    uint32_t pos_end = p.pos_end;
    if (p.live_blocks != nullptr) pos_end = min(pos_end, *p.n_live);
    const uint32_t pos_begin = min(p.pos_begin, pos_end);
    const uint32_t n_tiles = (pos_end - pos_begin + kConsumerWarps - 1) / kConsumerWarps;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], kConsumerWarps); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kConsumerWarps) {
        // ---------------- producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const uint32_t pos0 = pos_begin + tile * kConsumerWarps;
                const int nb = int(min(uint32_t(kConsumerWarps), pos_end - pos0));
                for (int ch = 0; ch < n_chunks && ok; ++ch, ++it) {
                    const int s = it % kStages;
                    ok = mbar_wait(&empty_bar[s], ((it / kStages) & 1) ^ 1, p.cb.error);
                    if (!ok) break;
                    const int rows = min(kChunkRows, ng - ch * kChunkRows);
                    const uint32_t bytes = uint32_t(rows) * kLanes;
                    mbar_arrive_expect_tx(&full_bar[s], bytes * nb);
                    for (int w = 0; w < nb; ++w) {
                        const uint32_t blk = p.live_blocks ? p.live_blocks[pos0 + w] : pos0 + w;
                        const uint8_t *src = p.codes + (size_t(blk) * ng + size_t(ch) * kChunkRows) * kLanes;
                        bulk_copy_g2s(stage_mem + size_t(s) * kStageBytes + size_t(w) * kChunkRows * kLanes, src,
                                      bytes, &full_bar[s]);
                    }
                }
            }
            // Drain: every copy this thread issued has to land before the CTA's shared memory is released.
            // The consumers release each stage after reading it, so waiting for the ring to come back
            // empty covers all of them; the wait is bounded like every other.
            for (int d = 0; d < kStages && ok; ++d, ++it)
                ok = mbar_wait(&empty_bar[it % kStages], ((it / kStages) & 1) ^ 1, p.cb.error);
        }
        return;
    }

    // ---------------- consumers ----------------
    const int quad = lane >> 2, t = lane & 3;
    const uint32_t T[4] = {p.level_words[0], p.level_words[1], p.level_words[2], p.level_words[3]};
    const uint32_t Tp[2] = {p.level_words[2], p.level_words[3]};
    const uint32_t Tn[2] = {negate_bytes(p.level_words[0]), negate_bytes(p.level_words[1])};
    const uint4 *wfrag = reinterpret_cast<const uint4 *>(p.wfrag);
    uint32_t it = 0;
    for (uint32_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const uint32_t pos = pos_begin + tile * kConsumerWarps + warp;
        const bool have = pos < pos_end;
        int acc[MT][4][4];
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[m][j][e] = 0;
        int accn[SPLIT ? MT : 1][4][4];                       // the c < 8 half of the contraction, subtracted at the end
#pragma unroll
        for (int m = 0; m < (SPLIT ? MT : 1); ++m)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) accn[m][j][e] = 0;

        for (int ch = 0; ch < n_chunks; ++ch, ++it) {
            const int s = it % kStages;
            if (!mbar_wait(&full_bar[s], (it / kStages) & 1, p.cb.error)) return;
            if (have) {
                // lane L < 16 addresses matrix row L of the vector half 0..15, lane L >= 16 that of the half 16..31
                const uint32_t rows_addr = smem_addr(stage_mem + size_t(s) * kStageBytes + size_t(warp) * kChunkRows * kLanes) +
                                           uint32_t((((lane & 15) >> 2) + 4 * (lane & 3)) * kLanes + (lane >> 4) * 16);
                const int rows_here = min(kChunkRows, ng - ch * kChunkRows);
                const int ksteps = (rows_here + 15) / 16;
                // query fragments of this chunk's k-steps: one pointer per chunk, constant strides inside
                const uint4 *wf = wfrag + (size_t(ch) * (kChunkRows / 16) * p.mtiles_total + p.mtile_base) * 32 + lane;
                const size_t wf_step = size_t(p.mtiles_total) * 32;
                auto kstep = [&](int ks) {
                    // x[j] = the byte-groups of rows 16ks + t + {0, 4, 8, 12} (bytes 0..3) of vector 8j + quad: the
                    // load unit transposes, matrix row 4t + r being pointed at row t + 4r so that the k order of the
                    // query fragments holds
                    uint32_t x[4];
                    ldmatrix_x2_trans_b8(x, rows_addr + ks * (16 * kLanes));
                    uint32_t b0[4], b1[4], n0[SPLIT ? 4 : 1], n1[SPLIT ? 4 : 1];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if constexpr (SPLIT) expand4_split(x[j], Tp, Tn, b0[j], b1[j], n0[j], n1[j]);
                        else expand4(x[j], T, b0[j], b1[j]);
                    }
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const uint4 a = __ldg(wf + ks * wf_step + m * 32);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            mma_s8(acc[m][j], a, b0[j], b1[j]);
                            if constexpr (SPLIT) mma_s8(accn[m][j], a, n0[j], n1[j]);
                        }
                    }
                };
                if (ksteps == kChunkRows / 16) {               // a whole chunk: no loop control, constant offsets
#pragma unroll
                    for (int ks = 0; ks < kChunkRows / 16; ++ks) kstep(ks);
                } else {
                    for (int ks = 0; ks < ksteps; ++ks) kstep(ks);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
        }

        if (have) {
            const uint32_t blk = p.live_blocks ? p.live_blocks[pos] : pos;
            const int64_t base = int64_t(blk) * kLanes;
            // accumulator columns 2t, 2t+1 of n-tile j are vectors 8j + 2t and 8j + 2t + 1
            float vs[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int v = 8 * (e >> 1) + 2 * t + (e & 1);
                vs[e] = (base + v < p.n) ? p.vec_scales[base + v] : 0.0f;
            }
            uint32_t allow = 0xffffffffu;
            if (p.mask) allow = reinterpret_cast<const uint32_t *>(p.mask)[blk];
#pragma unroll
            for (int m = 0; m < MT; ++m) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int ql = 16 * (p.mtile_base + m) + quad + 8 * half;   // query within the prepared batch
                    if (ql >= p.q_base + p.nq) continue;
                    const float qs = p.qscale[ql], qb = p.qbias[ql];
                    const uint64_t thr = p.cb.thr[ql], lo = p.cb.lo ? p.cb.lo[ql] : 0ull;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            const int vl = 8 * j + 2 * t + c;
                            if (base + vl >= p.n || !((allow >> vl) & 1u)) continue;
                            const int isum = SPLIT ? acc[m][j][2 * half + c] - accn[SPLIT ? m : 0][j][2 * half + c] : acc[m][j][2 * half + c];
                            const float score = __fmul_rn(fmaf(float(isum), qs, qb), vs[2 * j + c]);
                            push_candidate(p.cb, ql, score, uint32_t(base + vl), thr, lo);
                        }
                    }
                }
            }
        }
    }
}

// =====================================================================================================
// LUT scan (2/3-bit, and every geometry the permute-dot family does not cover): CUDA cores.
// isum = sum_g U[g][byte>>4] + U[g][16 + (byte&15)] exactly; float epilogue per mode:
//   kModeLutMulAdd: (f32)isum * scale + bias                      (search.rs:1176)
//   kModeLutFlush : acc = bias; per 256 groups acc = fma(scale, (f32)isum_batch, acc)   (search.rs:1596)
// One warp per code block; the tables of up to kLutQueriesPerLaunch queries sit in shared memory (the four
// group rows a warp instruction touches are 32 consecutive words, so its lookups never conflict).
// =====================================================================================================
template <int NQ>
__global__ void __launch_bounds__(256) scan_lut_kernel(ScanParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int ng = p.ngroups;
    uint8_t *lut = smem_raw;                                  // [NQ][ng*32]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nq_here = min(NQ, p.nq);
    for (int q = 0; q < nq_here; ++q) {
        const uint4 *src = reinterpret_cast<const uint4 *>(p.luts + size_t(p.q_base + q) * p.lut_pitch);
        uint4 *dst = reinterpret_cast<uint4 *>(lut + size_t(q) * ng * 32);
        for (int i = tid; i < ng * 2; i += blockDim.x) dst[i] = src[i];
    }
    __syncthreads();
    uint32_t pos_end = p.pos_end;
    if (p.live_blocks != nullptr) pos_end = min(pos_end, *p.n_live);
    const uint32_t pos_begin = min(p.pos_begin, pos_end);
    float qs[NQ], qb[NQ];
    uint64_t thr[NQ], lo[NQ];
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
        const int ql = p.q_base + min(q, nq_here - 1);
        qs[q] = p.qscale[ql]; qb[q] = p.qbias[ql]; thr[q] = p.cb.thr[ql];
        lo[q] = p.cb.lo ? p.cb.lo[ql] : 0ull;
    }
    const int warps = blockDim.x >> 5;
    // A warp instruction reads 128 contiguous bytes = four group rows of the block: lane = (row r = lane / 8,
    // vectors 4 * (lane % 8) .. + 3).  Each lane sums its quarter of the groups for its four vectors; the
    // integer partial sums of the four lanes that share a vector quad are added by two shuffles (integer
    // addition: the order does not matter), then lane (quad, r) finishes vector 4 * quad + r.
    const int row = lane >> 3, quad = lane & 7;
    const int my_vec = 4 * quad + row;
    for (uint32_t pos = pos_begin + blockIdx.x * warps + warp; pos < pos_end; pos += gridDim.x * warps) {
        const uint32_t blk = p.live_blocks ? p.live_blocks[pos] : pos;
        const uint32_t *codes32 = reinterpret_cast<const uint32_t *>(p.codes + size_t(blk) * ng * kLanes) + lane;
        const int64_t slot = int64_t(blk) * kLanes + my_vec;
        float facc[NQ];
#pragma unroll
        for (int q = 0; q < NQ; ++q) facc[q] = qb[q];
        uint32_t total[NQ];
#pragma unroll
        for (int q = 0; q < NQ; ++q) total[q] = 0;
        for (int g0 = 0; g0 < ng; g0 += 256) {
            const int g1 = min(g0 + 256, ng);
            uint32_t isum[NQ][4];
#pragma unroll
            for (int q = 0; q < NQ; ++q)
#pragma unroll
                for (int j = 0; j < 4; ++j) isum[q][j] = 0;
#pragma unroll 4
            for (int g = g0 + row; g < g1; g += 4) {
                const uint32_t word = codes32[size_t(g - row) * 8];      // bytes of vectors 4*quad .. +3 in group g
                const int o = g * 32;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t byte = (word >> (8 * j)) & 255u;
#pragma unroll
                    for (int q = 0; q < NQ; ++q)
                        isum[q][j] += uint32_t(lut[q * ng * 32 + o + (byte >> 4)]) + uint32_t(lut[q * ng * 32 + o + 16 + (byte & 15)]);
                }
            }
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
                uint32_t mine = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t v = isum[q][j];
                    v += __shfl_xor_sync(kFullMask, v, 8);
                    v += __shfl_xor_sync(kFullMask, v, 16);
                    if (j == row) mine = v;
                }
                facc[q] = fmaf(qs[q], float(int(mine)), facc[q]);
                total[q] += mine;
            }
        }
        if (slot < p.n) {
            const bool allowed = !p.mask || ((p.mask[slot >> 6] >> (slot & 63)) & 1ull);
            if (allowed) {
                const float vs = p.vec_scales[slot];
#pragma unroll
                for (int q = 0; q < NQ; ++q) {
                    if (q >= nq_here) break;
                    const float pre = p.mode == kModeLutFlush ? facc[q]
                                                              : __fadd_rn(__fmul_rn(float(int(total[q])), qs[q]), qb[q]);
                    push_candidate(p.cb, p.q_base + q, __fmul_rn(pre, vs), uint32_t(slot), thr[q], lo[q]);
                }
            }
        }
    }
}

// =====================================================================================================
// Selection: one CTA per query merges the previous top-k with the new candidates in shared memory.
// With few entries it is a plain bitonic sort.  With many more entries than k it is a bitonic top-k: sort
// runs of m = 2^ceil(log2 k) (at least 32) entries in alternating directions, then repeatedly take the
// element-wise minimum of each ascending/descending pair of runs (the m smallest of the pair, as a bitonic
// sequence), drop the other half, and re-sort the survivors' runs with one bitonic merge pass; the work is
// about n (log^2 m / 4 + 2 log m) compare-exchanges instead of n log^2 n / 4.  `dense_count` > 0 means the
// scan wrote exactly that many candidates per query without counting them (first chunk, see scan_tc.cu).
// =====================================================================================================
__device__ __forceinline__ void compare_exchange(uint64_t *keys, int lo, int hi, bool ascending) {
    const uint64_t a = keys[lo], b = keys[hi];
    if ((a > b) == ascending) { keys[lo] = b; keys[hi] = a; }
}

__global__ void __launch_bounds__(256) select_kernel(CandidateBuffers cb, int sort_n, int dense_count) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint64_t *keys = reinterpret_cast<uint64_t *>(smem_raw);
    const int q = blockIdx.x, tid = threadIdx.x;
    const uint32_t raw = dense_count > 0 ? uint32_t(dense_count) : cb.cnt[q];
    const int ncand = int(min(raw, uint32_t(cb.cap)));
    if (tid == 0 && raw > uint32_t(cb.cap)) atomicExch(cb.overflow, 1u);
    // a dense first chunk has no earlier results to merge with: leaving them out keeps 4096 candidates in a
    // 4096-entry network instead of an 8192-entry one
    const int nprev = dense_count > 0 ? 0 : cb.k;
    const int total = nprev + ncand;
    // smallest power of two holding the entries
    int n2 = 32;
    while (n2 < total) n2 <<= 1;
    if (n2 > sort_n) n2 = sort_n;
    for (int i = tid; i < n2; i += blockDim.x) {
        uint64_t v = kEmptyKey;
        if (i < nprev) v = cb.topk[size_t(q) * cb.k + i];
        else if (i < total) v = cb.cand[size_t(q) * cb.cap + (i - nprev)];
        keys[i] = v;
    }
    __syncthreads();
    int m = 32;
    while (m < cb.k) m <<= 1;
    if (n2 <= 2 * m) m = n2;                                  // nothing to gain: full sort
    // runs of m entries, ascending where (index & m) == 0, descending otherwise (m == n2: one ascending run)
    for (int size = 2; size <= m; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = tid; i < n2 / 2; i += blockDim.x) {
                const int lo = 2 * i - (i & (stride - 1));
                compare_exchange(keys, lo, lo + stride, (lo & size) == 0);
            }
            __syncthreads();
        }
    }
    // halving rounds: live runs sit at multiples of `step` entries; run r pairs with run r + 1 (r even)
    for (int step = m; step * 2 <= n2 && m < n2; step <<= 1) {
        const int pairs = n2 / (2 * step);
        // minimum of entry j of the first run and entry j of the second: the first run keeps the m smallest
        for (int i = tid; i < pairs * m; i += blockDim.x) {
            const int pr = i / m, j = i - pr * m;
            const int lo = pr * 2 * step + j, hi = lo + step;
            const uint64_t a = keys[lo], b = keys[hi];
            if (b < a) keys[lo] = b;
        }
        __syncthreads();
        // the survivors are bitonic: one merge pass sorts them, alternating directions for the next round
        for (int stride = m >> 1; stride > 0; stride >>= 1) {
            for (int i = tid; i < pairs * (m / 2); i += blockDim.x) {
                const int pr = i / (m / 2), j = i - pr * (m / 2);
                const int lo = pr * 2 * step + 2 * j - (j & (stride - 1));
                compare_exchange(keys, lo, lo + stride, (pr & 1) == 0);
            }
            __syncthreads();
        }
    }
    for (int i = tid; i < cb.k; i += blockDim.x) cb.topk[size_t(q) * cb.k + i] = keys[i];
    if (tid == 0) {
        cb.thr[q] = keys[cb.k - 1];      // kEmptyKey until k results exist: everything still passes
        cb.cnt[q] = 0;
    }
}

__global__ void finalize_kernel(CandidateBuffers cb, int nq, const unsigned long long *n_allowed, int64_t n,
                                float *scores, int64_t *slots, uint32_t *k_eff_out, int out_stride_is_k) {
    unsigned long long allowed = n_allowed ? *n_allowed : (unsigned long long)n;
    const int k_eff = int(min((unsigned long long)cb.k, min((unsigned long long)n, allowed)));
    const int stride = out_stride_is_k ? cb.k : k_eff;
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i == 0) *k_eff_out = uint32_t(k_eff);
    if (i >= int64_t(nq) * cb.k) return;
    const int q = int(i / cb.k), j = int(i % cb.k);
    if (j >= k_eff) return;
    const uint64_t key = cb.topk[i];
    float s = -INFINITY;
    int64_t slot = 0;                     // (-inf, 0) padding as search.rs:4341-4352
    if (key != kEmptyKey) { s = desc_bits_to_score(uint32_t(key >> 32)); slot = int64_t(key & 0xffffffffu); }
    scores[size_t(q) * stride + j] = s;
    slots[size_t(q) * stride + j] = slot;
}

__global__ void advance_floor_kernel(const uint64_t *thr, uint64_t *lo, int nq) {
    const int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q < nq) lo[q] = thr[q] == kEmptyKey ? kEmptyKey : thr[q] + 1;
}

// =====================================================================================================
// Device-side id -> slot table of an id-mapped index: open addressing with linear probing over
// (u64 key, u32 slot) pairs, hash = the multiply-shift mix the reference's IdHasher uses
// (turbovec/src/id_map.rs:65-85).  The host tables stay the authority (ids never leave the host in results);
// this copy only serves large allowlists, whose resolution - one hash lookup per id, id_map.rs:670-683 - would
// otherwise run on host threads: the ids are uploaded once and one kernel turns them into mask bits.
// =====================================================================================================
constexpr uint64_t kIdEmpty = 0xffffffffffffffffull, kIdTomb = 0xfffffffffffffffeull;
__device__ __forceinline__ uint32_t id_hash(uint64_t id, int log2cap) { return uint32_t((id * 0x9E3779B97F4A7C15ull) >> (64 - log2cap)); }

// ids[i] -> slot first + i, for ids not yet in the table (a rebuild, or the rows of an add)
__global__ void idtab_insert_kernel(uint64_t *keys, uint32_t *vals, int log2cap, const uint64_t *ids, int64_t n, uint32_t first) {
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t id = ids[i];
    const uint32_t mask = (1u << log2cap) - 1u;
    uint32_t h = id_hash(id, log2cap);
    for (uint32_t probe = 0; probe <= mask; ++probe, h = (h + 1) & mask) {
        const unsigned long long prev = atomicCAS(reinterpret_cast<unsigned long long *>(&keys[h]), kIdEmpty, id);
        if (prev == kIdEmpty || prev == id) { vals[h] = first + uint32_t(i); return; }
    }
}
// (id, slot) pairs with distinct ids: slot == 0xffffffff removes the id, otherwise sets (or inserts) its slot
__global__ void idtab_upsert_kernel(uint64_t *keys, uint32_t *vals, int log2cap, const uint64_t *ids, const uint32_t *slots, int64_t n) {
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t id = ids[i];
    const uint32_t slot = slots[i], mask = (1u << log2cap) - 1u;
    uint32_t h = id_hash(id, log2cap);
    for (uint32_t probe = 0; probe <= mask; ++probe, h = (h + 1) & mask) {
        const uint64_t k = keys[h];
        if (k == id) {
            if (slot == 0xffffffffu) keys[h] = kIdTomb; else vals[h] = slot;
            return;
        }
        if (k == kIdEmpty) {
            if (slot == 0xffffffffu) return;                  // removing an id that is not there
            const unsigned long long prev = atomicCAS(reinterpret_cast<unsigned long long *>(&keys[h]), kIdEmpty, id);
            if (prev == kIdEmpty) { vals[h] = slot; return; }
            // another new id took the place: keep probing
        }
    }
}
// allowlist ids -> mask bits; the smallest list index of an id that is not in the table goes to *first_unknown
__global__ void idtab_lookup_kernel(const uint64_t *keys, const uint32_t *vals, int log2cap, const uint64_t *ids, int64_t n,
                                    uint32_t *words32, unsigned long long *first_unknown) {
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t id = ids[i];
    const uint32_t mask = (1u << log2cap) - 1u;
    uint32_t h = id_hash(id, log2cap);
    for (uint32_t probe = 0; probe <= mask; ++probe, h = (h + 1) & mask) {
        const uint64_t k = keys[h];
        if (k == id) { const uint32_t s = vals[h]; atomicOr(&words32[s >> 5], 1u << (s & 31)); return; }
        if (k == kIdEmpty) break;
    }
    atomicMin(first_unknown, (unsigned long long)i);
}

// Keys of a finished search with a slot offset added (the shard's first global slot); empty entries stay empty.
__global__ void export_keys_kernel(const uint64_t *topk, int64_t count, uint64_t offset, uint64_t *out) {
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const uint64_t key = topk[i];
    out[i] = key == kEmptyKey ? key : key + offset;
}

// Merge of the per-shard result lists of one query: keys[list][q][k] -> the k best keys, decoded.  One CTA per
// query, bitonic sort of n_lists * k keys in shared memory (ascending keys = score descending, slot ascending).
// chunk_slots > 0: the lists hold LOCAL slots of shards that own chunks of that many slots round-robin (list r owns
// the chunks r, r + n_lists, ...); they become global slots before the sort, so ties break by the global slot.
__global__ void __launch_bounds__(256) merge_keys_kernel(const uint64_t *keys_in, int n_lists, int nq, int k, int n2,
                                                         uint32_t chunk_slots, float *scores, int64_t *slots) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint64_t *keys = reinterpret_cast<uint64_t *>(smem_raw);
    const int q = blockIdx.x, tid = threadIdx.x;
    const int total = n_lists * k;
    for (int i = tid; i < n2; i += blockDim.x) {
        uint64_t v = kEmptyKey;
        if (i < total) {
            v = keys_in[(size_t(i / k) * nq + q) * k + (i % k)];
            if (chunk_slots != 0 && v != kEmptyKey) {
                const uint32_t local = uint32_t(v), list = uint32_t(i / k);
                const uint64_t global = (uint64_t(local / chunk_slots) * uint32_t(n_lists) + list) * chunk_slots + local % chunk_slots;
                v = (v & 0xffffffff00000000ull) | global;
            }
        }
        keys[i] = v;
    }
    __syncthreads();
    for (int size = 2; size <= n2; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = tid; i < n2 / 2; i += blockDim.x) {
                const int lo = 2 * i - (i & (stride - 1));
                compare_exchange(keys, lo, lo + stride, (lo & size) == 0);
            }
            __syncthreads();
        }
    }
    for (int j = tid; j < k; j += blockDim.x) {
        const uint64_t key = keys[j];
        float s = -INFINITY;
        int64_t slot = 0;                 // (-inf, 0) padding, as finalize_kernel
        if (key != kEmptyKey) { s = desc_bits_to_score(uint32_t(key >> 32)); slot = int64_t(key & 0xffffffffu); }
        scores[size_t(q) * k + j] = s;
        slots[size_t(q) * k + j] = slot;
    }
}

}  // namespace

// =====================================================================================================
// Host launchers
// =====================================================================================================
size_t query_prep_smem_bytes(int dim) { return size_t(2) * (dim + 8) * 4 + size_t(dim) * 4; }

cudaError_t launch_query_prep(const QueryPrepParams &p, cudaStream_t stream) {
    if (p.nq <= 0) return cudaSuccess;
    const size_t smem = query_prep_smem_bytes(p.dim);
#define TV_LAUNCH_QP(L)                                                                                        \
    case L: {                                                                                                  \
        cudaError_t e = cudaFuncSetAttribute(query_prep_kernel<L>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                             int(smem));                                                       \
        if (e != cudaSuccess) return e;                                                                        \
        query_prep_kernel<L><<<p.nq, 128, smem, stream>>>(p);                                                  \
        break;                                                                                                 \
    }
    switch (rotation_variant(p.dim)) {
        TV_LAUNCH_QP(3) TV_LAUNCH_QP(4) TV_LAUNCH_QP(5) TV_LAUNCH_QP(6) TV_LAUNCH_QP(7)
        TV_LAUNCH_QP(8) TV_LAUNCH_QP(9) TV_LAUNCH_QP(10) TV_LAUNCH_QP(11) TV_LAUNCH_QP(12)
        default: return cudaErrorInvalidValue;
    }
#undef TV_LAUNCH_QP
    return cudaGetLastError();
}

cudaError_t launch_pack_bool_mask(const uint8_t *mask_bool, int64_t n, uint64_t *words, cudaStream_t s) {
    const int64_t padded = ((n + 63) / 64) * 64;
    if (padded == 0) return cudaSuccess;
    pack_bool_mask_kernel<<<unsigned((padded + 255) / 256), 256, 0, s>>>(mask_bool, n, reinterpret_cast<uint32_t *>(words));
    return cudaGetLastError();
}

cudaError_t launch_scatter_slots(const uint32_t *slots, int64_t count, uint64_t *words, cudaStream_t s) {
    if (count == 0) return cudaSuccess;
    scatter_slots_kernel<<<unsigned((count + 255) / 256), 256, 0, s>>>(slots, count, reinterpret_cast<uint32_t *>(words));
    return cudaGetLastError();
}

cudaError_t launch_mask_stats(uint64_t *words, int64_t n, unsigned long long *n_allowed, uint32_t *live_blocks,
                              uint32_t *n_live, cudaStream_t s) {
    const int64_t nblocks = (n + 31) / 32;
    if (nblocks == 0) return cudaSuccess;
    mask_stats_kernel<<<unsigned((nblocks + 255) / 256), 256, 0, s>>>(reinterpret_cast<uint32_t *>(words), n, n_allowed,
                                                                        live_blocks, n_live);
    return cudaGetLastError();
}

static int sort_capacity(int cap, int k) {
    int n2 = 32;
    while (n2 < cap + k) n2 <<= 1;
    return n2;
}
size_t select_smem_bytes(int cap, int k) { return size_t(sort_capacity(cap, k)) * 8; }

cudaError_t launch_select(const CandidateBuffers &cb, int nq, int dense_count, cudaStream_t s) {
    if (nq <= 0) return cudaSuccess;
    const int sort_n = sort_capacity(cb.cap, cb.k);
    const size_t smem = size_t(sort_n) * 8;
    // the attribute belongs to the current device: set on every launch (a host-side table write)
    cudaError_t e = cudaFuncSetAttribute(select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    select_kernel<<<nq, 256, smem, s>>>(cb, sort_n, dense_count);
    return cudaGetLastError();
}

cudaError_t launch_advance_floor(const uint64_t *thr, uint64_t *lo, int nq, cudaStream_t s) {
    if (nq <= 0) return cudaSuccess;
    advance_floor_kernel<<<(nq + 255) / 256, 256, 0, s>>>(thr, lo, nq);
    return cudaGetLastError();
}

cudaError_t launch_idtab_insert(uint64_t *keys, uint32_t *vals, int log2cap, const uint64_t *ids, int64_t n, uint32_t first, cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    idtab_insert_kernel<<<unsigned((n + 255) / 256), 256, 0, s>>>(keys, vals, log2cap, ids, n, first);
    return cudaGetLastError();
}
cudaError_t launch_idtab_upsert(uint64_t *keys, uint32_t *vals, int log2cap, const uint64_t *ids, const uint32_t *slots, int64_t n, cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    idtab_upsert_kernel<<<unsigned((n + 255) / 256), 256, 0, s>>>(keys, vals, log2cap, ids, slots, n);
    return cudaGetLastError();
}
cudaError_t launch_idtab_lookup(const uint64_t *keys, const uint32_t *vals, int log2cap, const uint64_t *ids, int64_t n, uint64_t *words,
                                unsigned long long *first_unknown, cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    idtab_lookup_kernel<<<unsigned((n + 255) / 256), 256, 0, s>>>(keys, vals, log2cap, ids, n, reinterpret_cast<uint32_t *>(words), first_unknown);
    return cudaGetLastError();
}

cudaError_t launch_export_keys(const uint64_t *topk, int64_t count, uint64_t offset, uint64_t *out, cudaStream_t s) {
    if (count <= 0) return cudaSuccess;
    export_keys_kernel<<<unsigned((count + 255) / 256), 256, 0, s>>>(topk, count, offset, out);
    return cudaGetLastError();
}

cudaError_t launch_merge_keys(const uint64_t *keys, int n_lists, int nq, int k, uint32_t chunk_slots, float *scores, int64_t *slots,
                              cudaStream_t s) {
    if (nq <= 0 || k <= 0 || n_lists <= 0) return cudaSuccess;
    int n2 = 32;
    while (n2 < n_lists * k) n2 <<= 1;
    if (n2 > kMergeMaxKeys) return cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(merge_keys_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMergeMaxKeys * 8);
    if (e != cudaSuccess) return e;
    merge_keys_kernel<<<nq, 256, size_t(n2) * 8, s>>>(keys, n_lists, nq, k, n2, chunk_slots, scores, slots);
    return cudaGetLastError();
}

cudaError_t launch_finalize(const CandidateBuffers &cb, int nq, const unsigned long long *n_allowed, int64_t n,
                            float *scores, int64_t *slots, uint32_t *k_eff_out, int out_stride_is_k, cudaStream_t s) {
    const int64_t total = int64_t(nq) * cb.k;
    finalize_kernel<<<unsigned((total + 255) / 256 + (total == 0)), 256, 0, s>>>(cb, nq, n_allowed, n, scores, slots,
                                                                                 k_eff_out, out_stride_is_k);
    return cudaGetLastError();
}

cudaError_t launch_scan_pd(const ScanParams &p, int sm_count, cudaStream_t s) {
    if (p.nq <= 0 || p.pos_end <= p.pos_begin) return cudaSuccess;
    const int mt = (p.nq + 15) / 16;
    const size_t smem = size_t(kStages) * kStageBytes;
    const uint32_t tiles = (p.pos_end - p.pos_begin + kConsumerWarps - 1) / kConsumerWarps;
    // the split lookup doubles the accumulators: with two query tiles the kernel needs 168 registers, one CTA per
    // SM, and is slower than the merged lookup (1.76 against 1.46 ms on 4 M vectors), so one tile only
    const bool split = p.pd_split != 0 && mt <= 1 && levels_split_ok(p.level_words);
    const unsigned per_sm = mt == 1 ? (split ? 2 : 3) : (mt == 2 ? 2 : 1);   // resident CTAs per SM (registers)
    const unsigned grid = unsigned(min(uint32_t(sm_count) * per_sm, tiles));
    const unsigned threads = (kConsumerWarps + 1) * 32;
#define TV_LAUNCH_PD(M, S)                                                                                          \
    {                                                                                                               \
        cudaError_t e = cudaFuncSetAttribute(scan_pd_kernel<M, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)); \
        if (e != cudaSuccess) return e;                                                                             \
        scan_pd_kernel<M, S><<<grid, threads, smem, s>>>(p);                                                        \
    }
    if (mt <= 1) { if (split) TV_LAUNCH_PD(1, true) else TV_LAUNCH_PD(1, false) }
    else if (mt <= 2) TV_LAUNCH_PD(2, false)
    else if (mt <= 4) TV_LAUNCH_PD(4, false)
    else return cudaErrorInvalidValue;
#undef TV_LAUNCH_PD
    return cudaGetLastError();
}

int scan_lut_width(int ngroups, size_t smem_limit) {
    const size_t table = size_t(ngroups) * 32;
    if (table == 0) return 0;
    const size_t fit = (smem_limit > 1024 ? smem_limit - 1024 : 0) / table;
    return fit >= 4 ? 4 : (fit >= 2 ? 2 : (fit >= 1 ? 1 : 0));
}

cudaError_t launch_scan_lut(const ScanParams &p, int sm_count, cudaStream_t s) {
    if (p.nq <= 0 || p.pos_end <= p.pos_begin) return cudaSuccess;
    if (p.nq > 4) return cudaErrorInvalidValue;
    // sized by the kernel's template width: its inner loop reads all NQ tables (unused ones hold garbage
    // whose sums are discarded), so the allocation must cover them
    const int width = p.nq == 1 ? 1 : (p.nq == 2 ? 2 : 4);
    const size_t smem = size_t(width) * p.ngroups * 32;
    const uint32_t blocks = p.pos_end - p.pos_begin;
    // resident CTAs per SM: as many as the tables leave room for (the scan hides its lookup latency with warps)
    const uint32_t per_sm = uint32_t(std::max<size_t>(1, std::min<size_t>(6, (size_t(200) << 10) / (smem + 1024))));
    const unsigned grid = unsigned(min(uint32_t(sm_count) * per_sm, (blocks + 7) / 8));
#define TV_LAUNCH_LUT(N)                                                                                             \
    {                                                                                                                \
        cudaError_t e = cudaFuncSetAttribute(scan_lut_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)); \
        if (e != cudaSuccess) return e;                                                                              \
        scan_lut_kernel<N><<<grid, 256, smem, s>>>(p);                                                               \
    }
    if (width == 1) TV_LAUNCH_LUT(1)
    else if (width == 2) TV_LAUNCH_LUT(2)
    else TV_LAUNCH_LUT(4)
#undef TV_LAUNCH_LUT
    return cudaGetLastError();
}

}  // namespace tv
