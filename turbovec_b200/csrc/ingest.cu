// Fused ingest kernel: per-vector norm -> rotation -> Lloyd-Max quantisation -> reconstruction inner
// product -> per-vector scale -> packing into the reference's 32-vector sequential-blocked layout.
//
// Reference path restated: encode::encode (turbovec/src/encode.rs:510-541) =
//   rotate_batch_into (:406-458; norm :920-932, zero-norm rule :446)
//   + encode_prerotated / fused_quantize_scale_pack_scalar (:560-652, :1418-1476)
//   + the blocked layout of pack.rs:340-361 (byte (block*ngroups + g)*32 + lane).
//
// Work decomposition.  One CTA owns one 32-slot code block and walks it in passes of V = blockDim/32
// vectors; warp w of a pass owns one vector.  Floating-point sums whose order the reference fixes are
// walked sequentially by one thread per chain (8 f32 chains for the norm, 4 f64 chains for the
// reconstruction inner product); everything else is data parallel across the warp.
#include "ingest.cuh"
#include "rotation.cuh"

namespace tv {
namespace {

struct IngestSmem {
    float *rowA;       // [V][stride]   input row, later the rotated row
    float *rowB;       // [V][stride]   intermediate of the rotation
    uint8_t *codes;    // [V][cstride]  one code per coordinate
    uint8_t *tile;     // [ngroups][V]  group bytes of this pass, lane-minor
    uint16_t *perm0, *perm1;
    float *norm, *inv;  // [V]
    double *cent64;    // [16]
    float *bnd;        // [15]
};

__device__ __forceinline__ IngestSmem carve(unsigned char *base, int V, int dim, int ngroups) {
    IngestSmem s;
    const int stride = dim + 8, cstride = dim + 4;
    size_t off = 0;
    s.cent64 = reinterpret_cast<double *>(base + off); off += 16 * sizeof(double);
    s.rowA = reinterpret_cast<float *>(base + off); off += size_t(V) * stride * 4;
    s.rowB = reinterpret_cast<float *>(base + off); off += size_t(V) * stride * 4;
    s.norm = reinterpret_cast<float *>(base + off); off += 8 * 4;
    s.inv = reinterpret_cast<float *>(base + off); off += 8 * 4;
    s.bnd = reinterpret_cast<float *>(base + off); off += 16 * 4;
    s.perm0 = reinterpret_cast<uint16_t *>(base + off); off += size_t(dim) * 2;
    s.perm1 = reinterpret_cast<uint16_t *>(base + off); off += size_t(dim) * 2;
    s.codes = base + off; off += size_t(V) * cstride;
    off = (off + 15) & ~size_t(15);
    s.tile = base + off;
    return s;
}

template <int LOG2B>
__global__ void __launch_bounds__(256) ingest_kernel(IngestParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int V = blockDim.x >> 5;
    const int dim = p.dim, ng = p.ngroups;
    const int stride = dim + 8, cstride = dim + 4;
    IngestSmem s = carve(smem_raw, V, dim, ng);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    for (int i = tid; i < dim; i += blockDim.x) { s.perm0[i] = p.perm0[i]; s.perm1[i] = p.perm1[i]; }
    const int nlev = 1 << p.bits;
    if (tid < nlev) s.cent64[tid] = double(p.centroids[tid]);
    if (tid < nlev - 1) s.bnd[tid] = p.boundaries[tid];

    const int64_t first_block = p.slot0 / kBlockLanes;
    const int64_t block = first_block + blockIdx.x;
    const int64_t slot_lo = p.slot0, slot_hi = p.slot0 + p.n;   // new rows occupy [slot_lo, slot_hi)
    const bool calibrated = p.shift != nullptr;
    const int cpb = 8 / p.bits;
    const int field = p.bits == 3 ? 4 : p.bits;
    __syncthreads();

    for (int pass = 0; pass * V < kBlockLanes; ++pass) {
        const int lane0 = pass * V;                       // first block lane of this pass
        const int64_t my_slot = block * kBlockLanes + lane0 + warp;
        const bool active = my_slot >= slot_lo && my_slot < slot_hi;
        // does any vector of this pass exist?
        const int64_t pass_lo = block * kBlockLanes + lane0, pass_hi = pass_lo + V;
        if (pass_hi <= slot_lo || pass_lo >= slot_hi) continue;   // uniform across the CTA

        float *rowA = s.rowA + size_t(warp) * stride;
        float *rowB = s.rowB + size_t(warp) * stride;
        uint8_t *codes = s.codes + size_t(warp) * cstride;

        // 1. load the row; flag the first non-finite / over-magnitude coordinate (encode.rs:58-74)
        if (active) {
            const int64_t row = my_slot - slot_lo;
            const float4 *src = reinterpret_cast<const float4 *>(p.x + row * dim);
            const int nvec = dim / 4;
            for (int i0 = lane; i0 < nvec; i0 += 32 * 4) {
                float4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {             // four loads in flight per lane before any use
                    const int i = i0 + 32 * u;
                    v[u] = i < nvec ? __ldcs(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = i0 + 32 * u;
                    if (i >= nvec) break;
                    reinterpret_cast<float4 *>(rowA)[i] = v[u];
                    const bool bx = !(fabsf(v[u].x) < kMaxMagnitude), by = !(fabsf(v[u].y) < kMaxMagnitude);
                    const bool bz = !(fabsf(v[u].z) < kMaxMagnitude), bw = !(fabsf(v[u].w) < kMaxMagnitude);
                    if (bx | by | bz | bw) {
                        const int c = bx ? 0 : by ? 1 : bz ? 2 : 3;
                        atomicMin(p.first_invalid, (unsigned long long)((p.row_base + row) * dim + 4 * i + c));
                    }
                }
            }
        }
        __syncthreads();

        // 2. norm: 8 sequential chains per vector, chain c sums x[j]^2 over j = c (mod 8), then the
        //    fixed tree ((c0+c1)+(c2+c3))+((c4+c5)+(c6+c7)) and a square root (encode.rs:900-932).
        if (tid < V * 8) {
            const int v = tid >> 3, c = tid & 7;
            const unsigned peers = V * 8 >= 32 ? kFullMask : ((1u << (V * 8)) - 1u);
            const float *row = s.rowA + size_t(v) * stride;
            float acc = 0.0f;
#pragma unroll 8
            for (int j = c; j < dim; j += 8) {
                const float x = row[j];
                acc = __fadd_rn(acc, __fmul_rn(x, x));
            }
            acc = __fadd_rn(acc, __shfl_down_sync(peers, acc, 1));    // valid on even c
            acc = __fadd_rn(acc, __shfl_down_sync(peers, acc, 2));    // valid on c % 4 == 0
            acc = __fadd_rn(acc, __shfl_down_sync(peers, acc, 4));    // valid on c == 0
            if (c == 0) {
                const float nv = __fsqrt_rn(acc);
                s.norm[v] = nv;
                s.inv[v] = nv > kMinNorm ? __fdiv_rn(1.0f, nv) : 0.0f;    // encode.rs:446
            }
        }
        __syncthreads();

        // 3. rotate (A -> B -> A), quantise, one code per coordinate
        if (p.rot_out != nullptr) {                       // rotate-only mode (uniform across the grid)
            if (active) {
                rotate_row<LOG2B>(rowA, rowB, s.perm0, s.perm1, dim, p.inv_sqrt_block, true, s.inv[warp], lane);
                float *out = p.rot_out + (my_slot - slot_lo) * dim;
                for (int j = lane; j < dim; j += 32) out[j] = rowA[j];
            }
            __syncthreads();
            continue;
        }
        if (active) {
            rotate_row<LOG2B>(rowA, rowB, s.perm0, s.perm1, dim, p.inv_sqrt_block, true, s.inv[warp], lane);
#pragma unroll 4
            for (int j = lane; j < dim; j += 32) {
                float calib = rowA[j];
                if (calibrated) calib = __fmul_rn(__fadd_rn(calib, p.shift[j]), p.scale_tq[j]);
                // number of boundaries strictly below calib (encode.rs:1447-1451); boundaries ascend
                int code = 0;
                for (int step = nlev >> 1; step >= 1; step >>= 1)
                    if (calib > s.bnd[code + step - 1]) code += step;
                codes[j] = uint8_t(code);
            }
        }
        __syncthreads();

        // 4. reconstruction inner product: 4 sequential f64 chains per vector, chain c over j = c (mod 4),
        //    combined as (c0+c1)+(c2+c3) (encode.rs:1418-1476); scale = norm / (f32)inner if inner > 0.1.
        if (tid < V * 4) {
            const int v = tid >> 2, c = tid & 3;
            const unsigned peers = V * 4 >= 32 ? kFullMask : ((1u << (V * 4)) - 1u);
            const float *row = s.rowA + size_t(v) * stride;
            const uint8_t *cd = s.codes + size_t(v) * cstride;
            const int64_t slot = block * kBlockLanes + lane0 + v;
            const bool live = slot >= slot_lo && slot < slot_hi;
            double acc = 0.0;
            if (!live) {
                // nothing to sum; the shuffles below still need this thread
            } else if (!calibrated) {
#pragma unroll 8
                for (int j = c; j < dim; j += 4)
                    acc = __dadd_rn(acc, __dmul_rn(double(row[j]), s.cent64[cd[j]]));
            } else {
                for (int j = c; j < dim; j += 4) {
                    const double recon = __dsub_rn(__dmul_rn(s.cent64[cd[j]], double(p.inv_scale_tq[j])),
                                                   double(p.shift[j]));        // encode.rs:276-278
                    acc = __dadd_rn(acc, __dmul_rn(double(row[j]), recon));
                }
            }
            acc = __dadd_rn(acc, __shfl_down_sync(peers, acc, 1));
            acc = __dadd_rn(acc, __shfl_down_sync(peers, acc, 2));
            if (c == 0 && live)
                p.scales[slot] = acc > 0.1 ? __fdiv_rn(s.norm[v], __double2float_rn(acc)) : 0.0f;
        }

       
        // 5. group bytes: coordinate g*cpb + k at shift (cpb-1-k)*field (pack.rs:264-282)
#pragma unroll 4
        for (int g = lane; g < ng; g += 32) {
            unsigned byte = 0;
            if (active)
                for (int k = 0; k < cpb; ++k) byte |= unsigned(codes[g * cpb + k]) << ((cpb - 1 - k) * field);
            s.tile[g * V + warp] = uint8_t(byte);
        }
        __syncthreads();

        // 6. store.  A pass whose V lanes are all new rows (or padding past the end of the index, which
        //    must read as zero) writes V-byte runs; a pass that shares its run with older rows writes
        //    only its own bytes.
        uint8_t *blk_base = p.codes + size_t(block) * ng * kBlockLanes;
        const bool whole = pass_lo >= slot_lo;   // nothing older in this run; lanes past slot_hi are zeros
        if (whole && V == 8) {
            for (int g = tid; g < ng; g += blockDim.x)
                *reinterpret_cast<uint2 *>(blk_base + size_t(g) * kBlockLanes + lane0) =
                    *reinterpret_cast<const uint2 *>(s.tile + g * 8);
        } else if (whole && V == 4) {
            for (int g = tid; g < ng; g += blockDim.x)
                *reinterpret_cast<uint32_t *>(blk_base + size_t(g) * kBlockLanes + lane0) =
                    *reinterpret_cast<const uint32_t *>(s.tile + g * 4);
        } else {
            for (int idx = tid; idx < ng * V; idx += blockDim.x) {
                const int g = idx / V, w = idx % V;
                const int64_t slot = pass_lo + w;
                if (slot >= slot_lo && (slot < slot_hi || whole))
                    blk_base[size_t(g) * kBlockLanes + lane0 + w] = s.tile[idx];
            }
        }
        __syncthreads();
    }
}

// Re-encoding of stored rows under a new TQ+ pair (reencode_stored_rows, turbovec/src/lib.rs:2760-2832), in
// place.  One warp per code block, lane = vector.  Pass 1 reconstructs the row from its codes under the
// committed pair, x[d] = centroids[code] * old_inv[d] - old_shift[d] (f32, two roundings), and sums x^2 in one
// f64 chain in coordinate order; the effective norm is (f64(scale_old) * sumsq) as f32.  Pass 2 is the fresh-row
// quantise + scale of encode_prerotated (encode.rs:560-652, 1418-1476) on that reconstruction under the new
// pair: four f64 chains over d % 4, (c0+c1)+(c2+c3), scale = norm / (f32)inner if inner > 0.1.
__global__ void __launch_bounds__(256) reencode_kernel(ReencodeParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t blk = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t slot = blk * kBlockLanes + lane;
    if (slot >= p.n) return;
    const int ng = p.ngroups, cpb = 8 / p.bits, field = p.bits == 3 ? 4 : p.bits;
    const uint32_t mask = (1u << p.bits) - 1u;
    const int nb = (1 << p.bits) - 1;
    uint8_t *codes = p.codes + size_t(blk) * ng * kBlockLanes + lane;
    double sumsq = 0.0;
    for (int g = 0; g < ng; ++g) {
        const uint32_t byte = codes[size_t(g) * kBlockLanes];
        for (int k = 0; k < cpb; ++k) {
            const int d = g * cpb + k;
            const uint32_t code = (byte >> ((cpb - 1 - k) * field)) & mask;
            const float inv = p.old_inv ? p.old_inv[d] : 1.0f, sh = p.old_shift ? p.old_shift[d] : 0.0f;
            const float x = __fsub_rn(__fmul_rn(p.centroids[code], inv), sh);
            sumsq = __dadd_rn(sumsq, __dmul_rn(double(x), double(x)));
        }
    }
    const float norm = __double2float_rn(__dmul_rn(double(p.scales[slot]), sumsq));
    double c0 = 0.0, c1 = 0.0, c2 = 0.0, c3 = 0.0;       // chain d % 4 (kept in registers: no indexed array)
    for (int g = 0; g < ng; ++g) {
        const uint32_t byte = codes[size_t(g) * kBlockLanes];
        uint32_t out = 0;
        for (int k = 0; k < cpb; ++k) {
            const int d = g * cpb + k;
            const uint32_t code = (byte >> ((cpb - 1 - k) * field)) & mask;
            const float inv = p.old_inv ? p.old_inv[d] : 1.0f, sh = p.old_shift ? p.old_shift[d] : 0.0f;
            const float x = __fsub_rn(__fmul_rn(p.centroids[code], inv), sh);
            const float nsh = p.new_shift[d];
            const float calib = __fmul_rn(__fadd_rn(x, nsh), p.new_scale[d]);
            uint32_t v = 0;
            for (int bi = 0; bi < nb; ++bi) v += calib > p.boundaries[bi] ? 1u : 0u;
            const double recon = __dsub_rn(__dmul_rn(double(p.centroids[v]), double(p.new_inv[d])), double(nsh));
            const double term = __dmul_rn(double(x), recon);
            switch (d & 3) {
                case 0: c0 = __dadd_rn(c0, term); break;
                case 1: c1 = __dadd_rn(c1, term); break;
                case 2: c2 = __dadd_rn(c2, term); break;
                default: c3 = __dadd_rn(c3, term); break;
            }
            out |= v << ((cpb - 1 - k) * field);
        }
        codes[size_t(g) * kBlockLanes] = uint8_t(out);
    }
    const double inner = __dadd_rn(__dadd_rn(c0, c1), __dadd_rn(c2, c3));
    p.scales[slot] = inner > 0.1 ? __fdiv_rn(norm, __double2float_rn(inner)) : 0.0f;
}

}  // namespace

size_t ingest_smem_bytes(int V, int dim, int ngroups) {
    size_t off = 16 * sizeof(double);
    off += size_t(2) * V * (dim + 8) * 4 + 16 * 4 + 16 * 4;
    off += size_t(dim) * 4;
    off += size_t(V) * (dim + 4);
    off = (off + 15) & ~size_t(15);
    off += size_t(ngroups) * V;
    return off;
}

int ingest_vectors_per_pass(int dim, int ngroups, size_t smem_limit) {
    // prefer 4 vectors per CTA so that several CTAs share an SM and hide the sequential chains
    for (int V : {4, 2, 1})
        if (ingest_smem_bytes(V, dim, ngroups) <= smem_limit) return V;
    return 0;
}

cudaError_t launch_ingest(const IngestParams &p, int V, cudaStream_t stream) {
    if (p.n <= 0) return cudaSuccess;
    const int64_t first_block = p.slot0 / kBlockLanes;
    const int64_t last_block = (p.slot0 + p.n - 1) / kBlockLanes;
    const unsigned grid = unsigned(last_block - first_block + 1);
    const size_t smem = ingest_smem_bytes(V, p.dim, p.ngroups);
    const int variant = rotation_variant(p.dim);
#define TV_LAUNCH_INGEST(L)                                                                               \
    case L: {                                                                                             \
        cudaError_t e = cudaFuncSetAttribute(ingest_kernel<L>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                             int(smem));                                                  \
        if (e != cudaSuccess) return e;                                                                   \
        ingest_kernel<L><<<grid, V * 32, smem, stream>>>(p);                                              \
        break;                                                                                            \
    }
    switch (variant) {
        TV_LAUNCH_INGEST(3) TV_LAUNCH_INGEST(4) TV_LAUNCH_INGEST(5) TV_LAUNCH_INGEST(6) TV_LAUNCH_INGEST(7)
        TV_LAUNCH_INGEST(8) TV_LAUNCH_INGEST(9) TV_LAUNCH_INGEST(10) TV_LAUNCH_INGEST(11) TV_LAUNCH_INGEST(12)
        default: return cudaErrorInvalidValue;
    }
#undef TV_LAUNCH_INGEST
    return cudaGetLastError();
}

cudaError_t launch_reencode(const ReencodeParams &p, cudaStream_t stream) {
    if (p.n <= 0) return cudaSuccess;
    const int64_t blocks = (p.n + kBlockLanes - 1) / kBlockLanes;
    reencode_kernel<<<unsigned((blocks + 7) / 8), 256, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace tv
