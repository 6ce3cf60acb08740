// Permute-dot scan for a handful of queries (up to 16): the HBM-bound form.
//
// Same arithmetic as scan_pd_kernel (search.cu): S[q][v] = sum_d W[q][d] * level[code[v][d]] exactly in int32
// (turbovec/src/search.rs:1392-1543), then fma((f32)S, scale_q, bias_q) * vec_scale[v] (search.rs:1523, 1793).
//
// What differs is the shape of the work.  With one query the scan streams 768 bytes per vector and does almost
// no arithmetic, so the kernel is built around the stream:
//   * the VECTORS sit on the M = 16 side of mma.sync.m16n8k32 and the queries on the N = 8 side, so one code block
//     (32 vectors) takes 2 MMAs per k-step and level half instead of 4, and 16 accumulator registers instead of 32;
//   * every warp owns a code block and is its own producer: a private ring of shared-memory stages filled by bulk
//     asynchronous copies that lane 0 issues (no producer warp, no barrier shared between warps, so warps drift
//     apart and overlap each other's load, lookup and MMA phases);
//   * the query operand is staged once per CTA in shared memory in fragment order (one 8-byte load per k-step);
//   * the level lookup is the split form of search.cu (two half-tables, two exact contractions, subtracted at the
//     end), which needs a codebook whose lower eight levels are <= 0 and upper eight >= 0.
// Thread t of a quad takes the byte-groups 4t .. 4t+3 of a k-step (16 byte-groups = 32 coordinates), so the eight
// row addresses of one phase of the transposing matrix load are eight consecutive 32-byte rows.
//
// Every wait is bounded.  A warp whose wait runs out records the error, waits (bounded again) for the other copies
// it has in flight and leaves; warps do not wait on one another after the prologue.
#include <cuda.h>

#include "scan_common.cuh"

namespace tv {
namespace {

constexpr int kSmallWarps = 8;                                 // warps (= code blocks in flight) per CTA
constexpr int kSmallChunkRows = 64;                            // byte-group rows per stage
constexpr int kSmallStageBytes = kSmallChunkRows * 32;         // 2 KB

__device__ __forceinline__ void tma_load_2d_small(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(x), "r"(y) : "memory");
}

// NT = query tiles of 8 (1 or 2).  STAGES = ring depth per warp.  SWZ: stages are filled by a tiled tensor copy with
// the 128-byte swizzle (four byte-group rows per 128-byte line), which makes every phase of the matrix load touch
// all 32 banks; otherwise by plain bulk copies (rows 32 bytes apart: two rows of a phase share a bank group).
template <int NT, int STAGES, bool SWZ, int CTAS>
__global__ void __launch_bounds__(kSmallWarps * 32, CTAS)
scan_small_kernel(ScanParams p, const int8_t *__restrict__ weights, int pitch, const __grid_constant__ CUtensorMap cmap) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ uint64_t full_bar[kSmallWarps][STAGES];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ng = p.ngroups;
    const int n_chunks = (ng + kSmallChunkRows - 1) / kSmallChunkRows;
    const int ksteps_total = (ng + 15) / 16;
    unsigned char *ring = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint2 *qfrag = reinterpret_cast<uint2 *>(ring + size_t(kSmallWarps) * STAGES * kSmallStageBytes);   // [NT][ksteps][32]

    uint32_t pos_end = p.pos_end;
    if (p.live_blocks != nullptr) pos_end = min(pos_end, *p.n_live);
    const uint32_t pos_begin = min(p.pos_begin, pos_end);

    if (tid == 0) {
        for (int w = 0; w < kSmallWarps; ++w)
            for (int s = 0; s < STAGES; ++s) mbar_init(&full_bar[w][s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Query operand in fragment order: lane (q, t) of k-step ks reads the weights of query q for the byte-groups
    // 16ks + 4t .. + 3, i.e. eight consecutive bytes of the query's row (the rows are stored with adjacent
    // coordinates swapped, which is the nibble order of a code byte: low nibble = odd coordinate).
    const int dim = ng * 2;
    for (int i = tid; i < NT * ksteps_total * 32; i += blockDim.x) {
        const int l = i & 31, ks = (i >> 5) % ksteps_total, nt = (i >> 5) / ksteps_total;
        const int q = nt * 8 + (l >> 2), off = 32 * ks + 8 * (l & 3);
        uint2 v = make_uint2(0u, 0u);
        if (q < p.nq && off < dim) {                           // dim is a multiple of 8: a group of eight bytes is whole
            v = *reinterpret_cast<const uint2 *>(weights + size_t(p.q_base + q) * pitch + off);
        }
        qfrag[i] = v;
    }
    __syncthreads();

    const int quad = lane >> 2, t = lane & 3;
    const uint32_t Tp[2] = {p.level_words[2], p.level_words[3]};
    const uint32_t Tn[2] = {negate_bytes(p.level_words[0]), negate_bytes(p.level_words[1])};
    const uint32_t total_warps = gridDim.x * kSmallWarps;
    const uint32_t gw = blockIdx.x * kSmallWarps + warp;
    const uint32_t n_pos = pos_end - pos_begin;
    const uint32_t my_blocks = gw < n_pos ? (n_pos - gw + total_warps - 1) / total_warps : 0;
    const uint32_t n_items = my_blocks * uint32_t(n_chunks);
    unsigned char *my_ring = ring + size_t(warp) * STAGES * kSmallStageBytes;
    uint64_t *my_bar = full_bar[warp];

    // per-query constants of this lane: queries 8nt + 2t and 8nt + 2t + 1
    float qs[NT][2], qb[NT][2];
    uint64_t thr[NT][2], lo[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int q = 8 * nt + 2 * t + c;
            const bool on = q < p.nq;
            qs[nt][c] = on ? p.qscale[p.q_base + q] : 0.f;
            qb[nt][c] = on ? p.qbias[p.q_base + q] : 0.f;
            thr[nt][c] = on ? p.cb.thr[p.q_base + q] : 0ull;   // 0: nothing passes
            lo[nt][c] = on && p.cb.lo ? p.cb.lo[p.q_base + q] : 0ull;
        }

    // ---- producer side (lane 0): item i = (block i / n_chunks of this warp, chunk i % n_chunks) ----
    uint32_t f_item = 0, f_pos = pos_begin + gw;
    int f_chunk = 0;
    auto issue = [&]() {
        if (f_item < n_items) {
            const int s = f_item % STAGES;
            const uint32_t blk = p.live_blocks ? p.live_blocks[f_pos] : f_pos;
            const int rows = min(kSmallChunkRows, ng - f_chunk * kSmallChunkRows);
            unsigned char *dst = my_ring + size_t(s) * kSmallStageBytes;
            if constexpr (SWZ) {
                // lines of 128 bytes = four byte-group rows; a box is 16 lines.  Lines past the block's end belong to
                // the next block (or are filled with zeros past the array): they meet zero weights.
                mbar_arrive_expect_tx(&my_bar[s], kSmallStageBytes);
                tma_load_2d_small(dst, &cmap, 0, int((size_t(blk) * ng + size_t(f_chunk) * kSmallChunkRows) >> 2), &my_bar[s]);
            } else {
                const uint32_t bytes = uint32_t(rows) * 32u;
                mbar_arrive_expect_tx(&my_bar[s], bytes);
                bulk_copy_g2s(dst, p.codes + (size_t(blk) * ng + size_t(f_chunk) * kSmallChunkRows) * 32, bytes, &my_bar[s]);
            }
        }
        ++f_item;
        if (++f_chunk == n_chunks) { f_chunk = 0; f_pos += total_warps; }
    };
    if (lane == 0)
        for (int s = 0; s < STAGES; ++s) issue();

    // row addresses of the matrix load.  Lanes 0..15 address matrix 0 = vectors 0..15, lanes 16..31 matrix 1 =
    // vectors 16..31; matrix row r = byte-group row r of the k-step.  Swizzled stages: 16-byte chunk c of line R
    // sits at chunk position c ^ (R % 8).
    uint32_t row_off0, row_off1;                               // this lane's row within an even / odd k-step
    {
        const int r = lane & 15, h = lane >> 4;
        if constexpr (SWZ) {
            // a k-step is 16 rows = 4 lines; line 4ks + R of the stage, so (line % 8) is R or R + 4 by the k-step's parity
            const int R = r >> 2, c = (r & 3) * 2 + h;
            row_off0 = uint32_t(R * 128 + ((c ^ R) << 4));
            row_off1 = uint32_t(R * 128 + ((c ^ (R + 4)) << 4));
        } else {
            row_off0 = row_off1 = uint32_t(r * 32 + h * 16);
        }
    }
    auto row_addr = [&](uint32_t stage_addr, int ks) -> uint32_t {
        return stage_addr + uint32_t(ks * 512) + ((ks & 1) ? row_off1 : row_off0);
    };

    bool ok = true;
    uint32_t it = 0;
    uint32_t pos = pos_begin + gw;
    for (uint32_t b = 0; b < my_blocks && ok; ++b, pos += total_warps) {
        const uint32_t blk = p.live_blocks ? p.live_blocks[pos] : pos;
        const int64_t base = int64_t(blk) * kLanes;
        // per-vector inputs of the epilogue, requested now so that they have arrived when the block is done:
        // accumulator rows quad and quad + 8 of tile m are the vectors 16m + quad and 16m + 8 + quad
        float vs[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int v = 16 * (e >> 1) + 8 * (e & 1) + quad;
            vs[e] = (base + v < p.n) ? __ldg(p.vec_scales + base + v) : 0.0f;
        }
        uint32_t allow = 0xffffffffu;
        if (p.mask) allow = __ldg(reinterpret_cast<const uint32_t *>(p.mask) + blk);

        int accp[NT][2][4], accn[NT][2][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int m = 0; m < 2; ++m)
#pragma unroll
                for (int e = 0; e < 4; ++e) { accp[nt][m][e] = 0; accn[nt][m][e] = 0; }

        for (int ch = 0; ch < n_chunks; ++ch, ++it) {
            const int s = it % STAGES;
            // warp-uniform outcome: the matrix load below is a warp-wide instruction
            if (!__all_sync(kFullMask, mbar_wait(&my_bar[s], (it / STAGES) & 1, p.cb.error))) { ok = false; break; }
            const uint32_t stage_addr = smem_addr(my_ring + size_t(s) * kSmallStageBytes);
            const int rows_here = min(kSmallChunkRows, ng - ch * kSmallChunkRows);
            const int ksteps = (rows_here + 15) / 16;
            const uint2 *qf = qfrag + size_t(ch) * (kSmallChunkRows / 16) * 32 + lane;
            auto kstep = [&](int ks) {
                // x[2i + h] = byte-groups 4t .. 4t+3 of this k-step for vector 16i + 8h + quad
                uint32_t x[4];
                ldmatrix_x2_trans_b8(x, row_addr(stage_addr, ks));
                uint32_t lp[4], hp[4], ln[4], hn[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) expand4_split(x[j], Tp, Tn, lp[j], hp[j], ln[j], hn[j]);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint2 w = qf[(size_t(nt) * ksteps_total + ks) * 32];
#pragma unroll
                    for (int m = 0; m < 2; ++m) {
                        // A rows quad / quad + 8 = vectors 16m + quad / 16m + 8 + quad; k halves = low / high selectors
                        mma_s8(accp[nt][m], make_uint4(lp[2 * m], lp[2 * m + 1], hp[2 * m], hp[2 * m + 1]), w.x, w.y);
                        mma_s8(accn[nt][m], make_uint4(ln[2 * m], ln[2 * m + 1], hn[2 * m], hn[2 * m + 1]), w.x, w.y);
                    }
                }
            };
            if (ksteps == kSmallChunkRows / 16) {
#pragma unroll
                for (int ks = 0; ks < kSmallChunkRows / 16; ++ks) kstep(ks);
            } else {
                for (int ks = 0; ks < ksteps; ++ks) kstep(ks);
            }
            __syncwarp();                                      // every lane has read the stage
            if (lane == 0) issue();                            // refill it with the chunk STAGES ahead
        }
        if (!ok) break;

        // ---- epilogue: accumulator (row, column) = (vector, query) ----
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int m = 0; m < 2; ++m)
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const int vl = 16 * m + 8 * hrow + quad;
                    if (base + vl >= p.n || !((allow >> vl) & 1u)) continue;
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int q = 8 * nt + 2 * t + c;
                        if (q >= p.nq) continue;
                        const int isum = accp[nt][m][2 * hrow + c] - accn[nt][m][2 * hrow + c];
                        const float score = __fmul_rn(fmaf(float(isum), qs[nt][c], qb[nt][c]), vs[2 * m + hrow]);
                        push_candidate(p.cb, p.q_base + q, score, uint32_t(base + vl), thr[nt][c], lo[nt][c]);
                    }
                }
    }
    if (!ok) {
        // a wait ran out: let the copies this warp still has in flight land before its CTA can retire
        for (uint32_t j = it + 1; j < min(n_items, it + uint32_t(STAGES)); ++j)
            mbar_wait(&my_bar[j % STAGES], (j / STAGES) & 1, p.cb.error);
    }
}

size_t small_smem_bytes(int nt, int stages, int ngroups) {
    return 1024 + size_t(kSmallWarps) * stages * kSmallStageBytes + size_t(nt) * ((ngroups + 15) / 16) * 256;
}

template <int NT, int STAGES, bool SWZ, int CTAS>
cudaError_t launch_variant(const ScanParams &p, const int8_t *weights, int pitch, const CUtensorMap &map, int sm_count,
                           cudaStream_t s) {
    const size_t smem = small_smem_bytes(NT, STAGES, p.ngroups);
    auto kern = scan_small_kernel<NT, STAGES, SWZ, CTAS>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
    const uint32_t blocks = p.pos_end - p.pos_begin;
    const unsigned grid = unsigned(min(uint32_t(sm_count) * CTAS, (blocks + kSmallWarps - 1) / kSmallWarps));
    kern<<<grid, kSmallWarps * 32, smem, s>>>(p, weights, pitch, map);
    return cudaGetLastError();
}

}  // namespace

bool scan_small_supported(const ScanParams &p, int nq_total, size_t smem_limit) {
    if (p.mode != kModePermuteDot || nq_total > 16 || p.ngroups % 4 != 0) return false;
    if (!levels_split_ok(p.level_words)) return false;
    return small_smem_bytes(nq_total > 8 ? 2 : 1, 3, p.ngroups) + 1024 <= smem_limit;
}

// variant: bits 0-1 = ring depth (0: 3 stages x 3 CTAs per SM, 1: 4 x 2, 2: 6 x 2), bit 2 = swizzled tensor copies.
cudaError_t launch_scan_small(const ScanParams &p, const int8_t *weights, int pitch, size_t code_bytes_capacity, int variant,
                              int sm_count, size_t smem_limit, cudaStream_t s) {
    if (p.nq <= 0 || p.pos_end <= p.pos_begin) return cudaSuccess;
    const bool swz = (variant & 4) != 0;
    CUtensorMap map{};
    if (swz) {
        typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                          const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                          CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
        EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(tensor_map_encoder());
        if (!enc) return cudaErrorNotSupported;
        const cuuint64_t dims[2] = {128, cuuint64_t(code_bytes_capacity / 128)};
        const cuuint64_t strides[1] = {128};
        const cuuint32_t box[2] = {128, cuuint32_t(kSmallStageBytes / 128)};
        const cuuint32_t estr[2] = {1, 1};
        if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(p.codes), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    const int nt = p.nq > 8 ? 2 : 1;
    int depth = variant & 3;
    // deeper rings need more shared memory: step down while the request exceeds the device's limit
    while (depth > 0 && small_smem_bytes(nt, depth == 1 ? 4 : 6, p.ngroups) + 1024 > smem_limit) --depth;
#define TV_SMALL(NT_, ST_, SW_, CT_) return launch_variant<NT_, ST_, SW_, CT_>(p, weights, pitch, map, sm_count, s)
    if (nt == 1) {
        if (!swz) { if (depth == 0) TV_SMALL(1, 3, false, 3); if (depth == 1) TV_SMALL(1, 4, false, 2); TV_SMALL(1, 6, false, 2); }
        else      { if (depth == 0) TV_SMALL(1, 3, true, 3);  if (depth == 1) TV_SMALL(1, 4, true, 2);  TV_SMALL(1, 6, true, 2); }
    } else {
        if (!swz) { if (depth == 0) TV_SMALL(2, 3, false, 2); if (depth == 1) TV_SMALL(2, 4, false, 2); TV_SMALL(2, 6, false, 2); }
        else      { if (depth == 0) TV_SMALL(2, 3, true, 2);  if (depth == 1) TV_SMALL(2, 4, true, 2);  TV_SMALL(2, 6, true, 2); }
    }
#undef TV_SMALL
}

}  // namespace tv
