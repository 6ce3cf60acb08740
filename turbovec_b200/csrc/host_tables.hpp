// Host-side one-off tables of the encode-and-scan path: the rotation's sign and
// permutation tables and the Lloyd-Max codebook.  Both are pure functions of
// (dim) resp. (bits, dim); they are computed once per index on the host and
// uploaded to the device.
#pragma once
#include <cstdint>
#include <vector>

namespace tv {

constexpr int kBlock = 32;               // vectors per code block      (turbovec/src/lib.rs:89)
constexpr int kFlushEvery = 256;         // byte-groups per LUT flush   (turbovec/src/lib.rs:102)
constexpr int kMaxDim = 16384;           // turbovec/src/lib.rs:101
constexpr float kMaxInputMagnitude = 1e16f;  // turbovec/src/lib.rs:109
constexpr float kMinInputNorm = 1e-10f;      // turbovec/src/lib.rs:163

struct RotationTables {
    int dim = 0;
    int block = 0;                       // largest power-of-two divisor of dim (rotation.rs:92-95)
    float inv_sqrt_block = 0.f;          // 1.0f / sqrtf(block)                  (rotation.rs:165)
    std::vector<float> signs[2];         // +1 / -1 per output slot and round
    std::vector<uint32_t> perms[2];      // perm[i] = source coordinate of output slot i
    // Device form: one u16 per output slot and round, low 15 bits = source index, bit 15 = sign is -1.
    std::vector<uint16_t> packed[2];
};

// turbovec/src/rotation.rs:141-187 (Rotation::new), :990-997 (fisher_yates).
RotationTables build_rotation_tables(int dim);

struct Codebook {
    std::vector<float> boundaries;       // 2^bits - 1, ascending
    std::vector<float> centroids;        // 2^bits, ascending
};

// turbovec/src/codebook.rs:69-167 (lloyd_max); memoised per (bits, dim) like codebook.rs:50-63.
const Codebook &codebook(int bits, int dim);

// Regularised incomplete beta I_x(a, b) (stands in for statrs 0.17.1 Beta::cdf).
double beta_cdf(double a, double b, double x);

}  // namespace tv
