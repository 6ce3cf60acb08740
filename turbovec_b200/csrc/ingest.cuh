// Launch interface of the fused ingest kernel (see ingest.cu).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <vector>

namespace tv {

constexpr int kBlockLanes = 32;              // vectors per code block (turbovec/src/lib.rs:89)
constexpr float kMaxMagnitude = 1e16f;       // turbovec/src/lib.rs:109
constexpr float kMinNorm = 1e-10f;           // turbovec/src/lib.rs:163

struct IngestParams {
    const float *x;                // [n][dim] device, row-major
    int64_t n;                     // rows in this batch
    int64_t slot0;                 // slot of the first row (= index length before the add)
    int64_t row_base;              // index of x's first row within the caller's whole batch (for error reports)
    int dim, bits, ngroups;
    const uint16_t *perm0, *perm1; // packed rotation tables (host_tables.hpp)
    float inv_sqrt_block;
    const float *boundaries;       // 2^bits - 1
    const float *centroids;        // 2^bits
    const float *shift;            // TQ+ pair or nullptr (identity)
    const float *scale_tq;
    const float *inv_scale_tq;     // 1.0f / scale_tq[d], rounded once in f32 (encode.rs:593)
    uint8_t *codes;                // sequential-blocked code array of the whole index
    float *scales;                 // per-slot scales of the whole index
    float *rot_out;                // when set: write the rotated unit rows [n][dim] here and encode nothing
                                   // (input of the TQ+ fit, encode.rs:470-480)
    unsigned long long *first_invalid;  // min flat index of a coordinate failing |x| < 1e16 (init ~0ull)
    int exact_sums;                // pipelined kernel only: 1 = always walk the reference's sequential f64 chains (testing)
    const uint8_t *store_bank;     // pipelined kernel only: exchange layout (ExchangeLayoutHost), or nullptr = linear rows
    const uint16_t *perm1_exchange;
};

size_t ingest_smem_bytes(int vectors_per_pass, int dim, int ngroups);
// Largest supported vectors-per-pass whose shared memory fits `smem_limit`, 0 if none.
int ingest_vectors_per_pass(int dim, int ngroups, size_t smem_limit);
cudaError_t launch_ingest(const IngestParams &p, int vectors_per_pass, cudaStream_t stream);

// Stored rows re-encoded in place under a new TQ+ pair (see reencode_kernel in ingest.cu).
struct ReencodeParams {
    uint8_t *codes;                // sequential-blocked code array of the whole index
    float *scales;
    int64_t n;
    int dim, bits, ngroups;
    const float *boundaries, *centroids;
    const float *old_shift, *old_inv;          // committed pair (1 / scale rounded in f32), or nullptr = identity
    const float *new_shift, *new_scale, *new_inv;
};
cudaError_t launch_reencode(const ReencodeParams &p, cudaStream_t stream);
// Two order statistics per column of a rows x dim matrix on the device (quantile.cu): the TQ+ fit's quantiles.
cudaError_t launch_quantile_pair(const float *rot, int64_t n, int dim, int64_t lo_rank, int64_t hi_rank, float *q_lo, float *q_hi,
                                 cudaStream_t stream);

// Pipelined form (ingest_fast.cu) for whole code blocks: p.slot0 a multiple of 32, no calibration, no
// rotate-only mode, x 16-byte aligned, dim one of the instantiated sizes, shared memory within the limit.
// It quantises through a grid table built once per codebook: cell c holds the number of boundaries in lower
// cells (times 8) and the one boundary inside the cell (f32 bits; FLT_MAX when there is none).
struct QuantCell { uint32_t boundary_bits, code8; };
struct QuantGridHost {
    float a = 0.f, b = 0.f;              // cell of x = f(sat(x * a + b)), see grid_offset
    std::vector<QuantCell> cells;        // 1024 entries
};
struct QuantGrid {                       // device view, passed to the kernel by value
    const uint2 *cells = nullptr;
    float a = 0.f, b = 0.f;
};
// False when two boundaries share a cell or the boundaries are not strictly ascending and finite; the
// caller then keeps to launch_ingest.
bool build_quant_grid(const float *boundaries, int count, QuantGridHost &out);
uint32_t quant_grid_code(const QuantGridHost &grid, float x);   // host evaluation, the kernel's lookup
// Conflict-free layout of the row through which the two rotation rounds of the pipelined kernel exchange
// data (built once per dimension, see ingest_fast.cu): byte offset within its 128-byte row of every stored
// register [k*32 + lane], and the round-2 table with source positions in that layout (same packing as perm1).
struct ExchangeLayoutHost {
    int T = 0;
    std::vector<uint8_t> store_bank;
    std::vector<uint16_t> perm1_exchange;
};
bool build_exchange_layout(int dim, const uint16_t *perm1_packed, ExchangeLayoutHost &out);
void exchange_layout_conflicts(int dim, const uint16_t *perm1_packed, const ExchangeLayoutHost *layout_or_null, int *store_max,
                               int *gather_max);
bool ingest_fast_supported(int dim, int bits, int ngroups, bool calibrated, const void *x, size_t smem_limit);
// `error` receives a non-zero code if a bounded wait inside the kernel gives up.
cudaError_t launch_ingest_fast(const IngestParams &p, const QuantGrid &grid, int sm_count, size_t smem_limit, uint32_t *error,
                               cudaStream_t stream);

}  // namespace tv
