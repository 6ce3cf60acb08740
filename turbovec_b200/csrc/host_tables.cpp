#include "host_tables.hpp"

#include <array>
#include <cmath>
#include <map>
#include <mutex>
#include <utility>

namespace tv {
namespace {

// ChaCha with 8 rounds as rand_chacha 0.3.1 exposes it: 256-bit key, 64-bit block counter in
// state words 12-13, stream id 0, output consumed as little-endian u32 words in order.
class ChaCha8Stream {
  public:
    explicit ChaCha8Stream(const std::array<uint8_t, 32> &seed) {
        for (int i = 0; i < 8; ++i)
            key_[i] = uint32_t(seed[4 * i]) | uint32_t(seed[4 * i + 1]) << 8 | uint32_t(seed[4 * i + 2]) << 16 |
                      uint32_t(seed[4 * i + 3]) << 24;
    }
    uint32_t next_u32() {
        if (pos_ == 16) refill();
        return out_[pos_++];
    }
    // rand_core's block-RNG next_u64: two consecutive words, low word first.
    uint64_t next_u64() {
        uint64_t lo = next_u32();
        uint64_t hi = next_u32();
        return hi << 32 | lo;
    }

  private:
    static uint32_t rotl(uint32_t v, int s) { return v << s | v >> (32 - s); }
    static void quarter(uint32_t *x, int a, int b, int c, int d) {
        x[a] += x[b]; x[d] = rotl(x[d] ^ x[a], 16);
        x[c] += x[d]; x[b] = rotl(x[b] ^ x[c], 12);
        x[a] += x[b]; x[d] = rotl(x[d] ^ x[a], 8);
        x[c] += x[d]; x[b] = rotl(x[b] ^ x[c], 7);
    }
    void refill() {
        uint32_t in[16] = {0x61707865u, 0x3320646eu, 0x79622d32u, 0x6b206574u};
        for (int i = 0; i < 8; ++i) in[4 + i] = key_[i];
        in[12] = uint32_t(counter_);
        in[13] = uint32_t(counter_ >> 32);
        in[14] = in[15] = 0;
        uint32_t x[16];
        for (int i = 0; i < 16; ++i) x[i] = in[i];
        for (int dr = 0; dr < 4; ++dr) {
            quarter(x, 0, 4, 8, 12); quarter(x, 1, 5, 9, 13); quarter(x, 2, 6, 10, 14); quarter(x, 3, 7, 11, 15);
            quarter(x, 0, 5, 10, 15); quarter(x, 1, 6, 11, 12); quarter(x, 2, 7, 8, 13); quarter(x, 3, 4, 9, 14);
        }
        for (int i = 0; i < 16; ++i) out_[i] = x[i] + in[i];
        ++counter_;
        pos_ = 0;
    }
    uint32_t key_[8];
    uint64_t counter_ = 0;
    uint32_t out_[16];
    int pos_ = 16;
};

// turbovec/src/rotation.rs:82-85
constexpr std::array<uint8_t, 32> kRotationSeed = {164, 143, 161, 123, 88,  50,  61,  10,  234, 184, 161,
                                                   204, 105, 1,   20,  184, 43,  140, 200, 117, 24,  180,
                                                   247, 84,  141, 68,  110, 161, 228, 223, 32,  242};

}  // namespace

RotationTables build_rotation_tables(int dim) {
    RotationTables t;
    t.dim = dim;
    t.block = dim & -dim;
    t.inv_sqrt_block = 1.0f / std::sqrt(float(t.block));
    ChaCha8Stream rng(kRotationSeed);
    for (int r = 0; r < 2; ++r) {
        t.signs[r].resize(dim);
        t.perms[r].resize(dim);
        for (int i = 0; i < dim; ++i) t.signs[r][i] = (rng.next_u32() & 1u) ? -1.0f : 1.0f;
        for (int i = 0; i < dim; ++i) t.perms[r][i] = uint32_t(i);
        for (int i = dim - 1; i >= 1; --i) {
            uint64_t j = rng.next_u64() % (uint64_t(i) + 1);
            std::swap(t.perms[r][i], t.perms[r][j]);
        }
        t.packed[r].resize(dim);
        for (int i = 0; i < dim; ++i)
            t.packed[r][i] = uint16_t(t.perms[r][i] | (t.signs[r][i] < 0.f ? 0x8000u : 0u));
    }
    return t;
}

// ---------------------------------------------------------------------------------------------
// Beta(a, a) on [0, 1] and the Lloyd-Max solver
// ---------------------------------------------------------------------------------------------
namespace {

// Evaluates the continued fraction of the incomplete beta function with the modified Lentz scheme.
double beta_fraction(double a, double b, double x) {
    constexpr double tiny = 1e-300, eps = 1e-16;
    const double sum = a + b, ap = a + 1.0, am = a - 1.0;
    double c = 1.0, d = 1.0 - sum * x / ap;
    if (std::fabs(d) < tiny) d = tiny;
    d = 1.0 / d;
    double f = d;
    for (int m = 1; m <= 100000; ++m) {
        const double tm = 2.0 * m;
        double num = m * (b - m) * x / ((am + tm) * (a + tm));
        d = 1.0 + num * d; if (std::fabs(d) < tiny) d = tiny;
        c = 1.0 + num / c; if (std::fabs(c) < tiny) c = tiny;
        d = 1.0 / d;
        f *= d * c;
        num = -(a + m) * (sum + m) * x / ((a + tm) * (ap + tm));
        d = 1.0 + num * d; if (std::fabs(d) < tiny) d = tiny;
        c = 1.0 + num / c; if (std::fabs(c) < tiny) c = tiny;
        d = 1.0 / d;
        const double step = d * c;
        f *= step;
        if (std::fabs(step - 1.0) < eps) break;
    }
    return f;
}

struct SymmetricBeta {
    double a, log_norm;  // log B(a, a)
    explicit SymmetricBeta(double a_) : a(a_), log_norm(2.0 * std::lgamma(a_) - std::lgamma(2.0 * a_)) {}
    double pdf(double t) const {
        if (t <= 0.0 || t >= 1.0) return 0.0;
        return std::exp((a - 1.0) * std::log(t) + (a - 1.0) * std::log1p(-t) - log_norm);
    }
};

// Integrand of the conditional mean on [-1, 1]: x * pdf((x+1)/2) / 2  (codebook.rs:114-117).
struct MeanIntegrand {
    const SymmetricBeta &beta;
    double operator()(double x) const { return x * beta.pdf((x + 1.0) / 2.0) / 2.0; }
};

// codebook.rs:225-249
double simpson_refine(const MeanIntegrand &f, double a, double b, double fa, double fb, double fm, double whole,
                      double tol, int depth) {
    const double mid = (a + b) / 2.0, m1 = (a + mid) / 2.0, m2 = (mid + b) / 2.0;
    const double fm1 = f(m1), fm2 = f(m2);
    const double left = (mid - a) / 6.0 * (fa + 4.0 * fm1 + fm);
    const double right = (b - mid) / 6.0 * (fm + 4.0 * fm2 + fb);
    const double refined = left + right;
    if (depth == 0 || std::fabs(refined - whole) < 15.0 * tol) return refined + (refined - whole) / 15.0;
    return simpson_refine(f, a, mid, fa, fm, fm1, left, tol / 2.0, depth - 1) +
           simpson_refine(f, mid, b, fm, fb, fm2, right, tol / 2.0, depth - 1);
}

// codebook.rs:214-223
double simpson(const MeanIntegrand &f, double a, double b, double tol, int depth) {
    const double mid = (a + b) / 2.0;
    const double fa = f(a), fb = f(b), fm = f(mid);
    return simpson_refine(f, a, b, fa, fb, fm, (b - a) / 6.0 * (fa + 4.0 * fm + fb), tol, depth);
}

Codebook solve_lloyd_max(int bits, int dim) {
    const double a = (double(dim) - 1.0) / 2.0;
    const SymmetricBeta beta(a);
    const MeanIntegrand integrand{beta};
    const int levels = 1 << bits;
    const double sigma = std::sqrt(2.0 * a / ((2.0 * a + 1.0) * 4.0 * a));
    const double spread = 3.0 * sigma;
    std::vector<double> cur(levels), next(levels), edges(levels + 1);
    for (int i = 0; i < levels; ++i) cur[i] = -spread + 2.0 * spread * double(i) / (double(levels) - 1.0);
    for (int iter = 0; iter < 200; ++iter) {
        edges[0] = -1.0;
        for (int i = 0; i + 1 < levels; ++i) edges[i + 1] = (cur[i] + cur[i + 1]) / 2.0;
        edges[levels] = 1.0;
        for (int i = 0; i < levels; ++i) {
            const double lo = edges[i], hi = edges[i + 1];
            const double mass = beta_cdf(a, a, (hi + 1.0) / 2.0) - beta_cdf(a, a, (lo + 1.0) / 2.0);
            next[i] = mass < 1e-15 ? cur[i] : simpson(integrand, lo, hi, 1e-14, 50) / mass;
        }
        double moved = 0.0;
        for (int i = 0; i < levels; ++i) moved = std::fmax(moved, std::fabs(cur[i] - next[i]));
        cur = next;
        if (moved < 1e-12) break;
    }
    Codebook cb;
    cb.centroids.resize(levels);
    cb.boundaries.resize(levels - 1);
    for (int i = 0; i < levels; ++i) cb.centroids[i] = float(cur[i]);
    // f32 midpoints of the f32 centroids (codebook.rs:159-164)
    for (int i = 0; i + 1 < levels; ++i) cb.boundaries[i] = (cb.centroids[i] + cb.centroids[i + 1]) * 0.5f;
    return cb;
}

}  // namespace

double beta_cdf(double a, double b, double x) {
    if (x <= 0.0) return 0.0;
    if (x >= 1.0) return 1.0;
    const double front = std::exp(std::lgamma(a + b) - std::lgamma(a) - std::lgamma(b) + a * std::log(x) +
                                  b * std::log1p(-x));
    if (x < (a + 1.0) / (a + b + 2.0)) return front * beta_fraction(a, b, x) / a;
    return 1.0 - front * beta_fraction(b, a, 1.0 - x) / b;
}

const Codebook &codebook(int bits, int dim) {
    static std::mutex mu;
    static std::map<std::pair<int, int>, Codebook> memo;
    std::lock_guard<std::mutex> lock(mu);
    auto key = std::make_pair(bits, dim);
    auto it = memo.find(key);
    if (it == memo.end()) it = memo.emplace(key, solve_lloyd_max(bits, dim)).first;
    return it->second;
}

}  // namespace tv
