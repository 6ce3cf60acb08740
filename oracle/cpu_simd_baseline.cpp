// CPU SIMD baseline for the benchmark's CPU arm: a C++ restatement of the reference's fastest x86 search
// kernel for 4-bit codes — permute-dot on the vector-major layout with AVX-512 VNNI
// (turbovec/src/search.rs:1392-1543; layout turbovec/src/pack.rs:1269-1271; weight order
// search.rs:2806-2846; heap update search.rs:1768-1852; tiling search.rs:3997-4046) — multithreaded over
// (query batch of 8) x (block range) tiles with a (score desc, slot asc) merge (search.rs:4285-4298).
//
// TEST / MEASUREMENT INFRASTRUCTURE ONLY, like the rest of this directory.  It exists so that the CPU
// number printed beside the GPU number is the reference's SIMD algorithm on all host cores rather than a
// scalar loop.  Its results are checked against the scalar oracle (tests/test_cpu_simd_baseline.py).
// On a host without AVX-512 VNNI tvs_available() returns 0 and the caller falls back to the scalar oracle.
#include <immintrin.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

constexpr int kBlock = 32;

struct Cand { float s; int64_t i; };
inline bool better(const Cand &a, const Cand &b) { return a.s > b.s || (a.s == b.s && a.i < b.i); }

struct TopK {
    std::vector<Cand> v; int k; float thr = -INFINITY;
    explicit TopK(int k_) : k(k_) { v.reserve(k_ + 1); }
    inline void push(float s, int64_t i) {
        Cand c{s, i};
        if (int(v.size()) == k) { if (!better(c, v.back())) return; v.pop_back(); }
        v.insert(std::upper_bound(v.begin(), v.end(), c, better), c);
        if (int(v.size()) == k) thr = v.back().s;
    }
};

__attribute__((target("avx512f,avx512bw,avx512vnni,avx2,fma")))
void scan_tile(const uint8_t *vm_codes, int quads, const float *vec_scales, int64_t n, int64_t b0, int64_t b1,
               const int8_t *levels, const int8_t *const *weights, const int32_t *zeros, const float *qscale,
               const float *qbias, int nqb, const uint64_t *mask, TopK *heaps) {
    const __m512i m0f = _mm512_set1_epi8(0x0F);
    const __m512i lv = _mm512_xor_si512(_mm512_broadcast_i32x4(_mm_loadu_si128((const __m128i *)levels)),
                                        _mm512_set1_epi8((char)0x80));       // +128: unsigned operand of vpdpbusd
    const size_t block_bytes = size_t(quads) * 128;
    for (int64_t b = b0; b < b1; ++b) {
        const int64_t base = b * kBlock;
        uint32_t allow = 0xffffffffu;
        if (mask) {
            allow = uint32_t(mask[base >> 6] >> (base & 63));
            if (!allow) continue;                                            // search.rs:3015-3029
        }
        __m512i acc[8][2];
        for (int q = 0; q < nqb; ++q) acc[q][0] = acc[q][1] = _mm512_set1_epi32(zeros[q]);
        const uint8_t *blk = vm_codes + size_t(b) * block_bytes;
        for (int q4 = 0; q4 < quads; ++q4) {
            for (int h = 0; h < 2; ++h) {
                const __m512i c = _mm512_loadu_si512(blk + size_t(q4) * 128 + h * 64);
                const __m512i vlo = _mm512_shuffle_epi8(lv, _mm512_and_si512(c, m0f));
                const __m512i vhi = _mm512_shuffle_epi8(lv, _mm512_and_si512(_mm512_srli_epi16(c, 4), m0f));
                for (int q = 0; q < nqb; ++q) {
                    int32_t wl, wh;
                    std::memcpy(&wl, weights[q] + q4 * 8, 4);
                    std::memcpy(&wh, weights[q] + q4 * 8 + 4, 4);
                    acc[q][h] = _mm512_dpbusd_epi32(acc[q][h], vlo, _mm512_set1_epi32(wl));
                    acc[q][h] = _mm512_dpbusd_epi32(acc[q][h], vhi, _mm512_set1_epi32(wh));
                }
            }
        }
        const int lanes = int(std::min<int64_t>(kBlock, n - base));
        for (int q = 0; q < nqb; ++q) {
            const __m512 vs = _mm512_set1_ps(qscale[q]), vb = _mm512_set1_ps(qbias[q]);
            alignas(64) float out[32];
            if (lanes == kBlock) {
                _mm512_store_ps(out, _mm512_mul_ps(_mm512_fmadd_ps(_mm512_cvtepi32_ps(acc[q][0]), vs, vb), _mm512_loadu_ps(vec_scales + base)));
                _mm512_store_ps(out + 16, _mm512_mul_ps(_mm512_fmadd_ps(_mm512_cvtepi32_ps(acc[q][1]), vs, vb), _mm512_loadu_ps(vec_scales + base + 16)));
            } else {
                alignas(64) float f[32];
                _mm512_store_ps(f, _mm512_fmadd_ps(_mm512_cvtepi32_ps(acc[q][0]), vs, vb));
                _mm512_store_ps(f + 16, _mm512_fmadd_ps(_mm512_cvtepi32_ps(acc[q][1]), vs, vb));
                for (int l = 0; l < lanes; ++l) out[l] = f[l] * vec_scales[base + l];
            }
            TopK &hp = heaps[q];
            for (int l = 0; l < lanes; ++l) {
                if (!((allow >> l) & 1u)) continue;
                if (out[l] >= hp.thr) hp.push(out[l], base + l);
            }
        }
    }
}

}  // namespace

extern "C" {

int tvs_available(void) {
    return __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") && __builtin_cpu_supports("avx512vnni");
}

// sequential-blocked -> vector-major (pack.rs:1269-1271): byte (g, lane) of a block goes to
// (g/4)*128 + (lane/16)*64 + (lane%16)*4 + g%4.  ngroups must be a multiple of 4.
void tvs_to_vector_major(const uint8_t *blocked, int64_t n_blocks, int ngroups, uint8_t *vm) {
    for (int64_t b = 0; b < n_blocks; ++b) {
        const uint8_t *src = blocked + size_t(b) * ngroups * kBlock;
        uint8_t *dst = vm + size_t(b) * ngroups * kBlock;
        for (int g = 0; g < ngroups; ++g)
            for (int l = 0; l < kBlock; ++l) dst[(g / 4) * 128 + (l / 16) * 64 + (l % 16) * 4 + (g % 4)] = src[g * kBlock + l];
    }
}

// Queries arrive prepared (rotated, int8 weights in coordinate order, per-query scale and bias), as the
// scalar oracle's tvo_query_tables produces them; this routine times only what the reference's scan times.
// Returns k_eff; writes nq*k_eff scores / slots.
int64_t tvs_search_pd(const uint8_t *vm_codes, const float *vec_scales, int64_t n, int dim, const int8_t *levels,
                      const int8_t *weights_coord, const float *qscale, const float *qbias, int64_t nq, int64_t k,
                      const uint64_t *mask, int n_threads, float *scores_out, int64_t *slots_out) {
    const int ng = dim / 2, quads = ng / 4;
    int64_t n_allowed = n;
    if (mask) { n_allowed = 0; for (int64_t w = 0; w < (n + 63) / 64; ++w) n_allowed += __builtin_popcountll(mask[w]); }
    k = std::min(k, n_allowed);
    if (k <= 0 || nq <= 0) return std::max<int64_t>(k, 0);
    const int64_t n_blocks = (n + kBlock - 1) / kBlock;
    // kernel weight order: per quad of 4 byte-groups, 4 low-nibble (odd coordinate) weights then 4 high-nibble ones
    std::vector<int8_t> wk(size_t(nq) * ng * 2);
    std::vector<int32_t> zeros(nq);
    for (int64_t q = 0; q < nq; ++q) {
        int32_t wsum = 0;
        for (int g = 0; g < ng; ++g) {
            const int8_t lo = weights_coord[q * dim + 2 * g + 1], hi = weights_coord[q * dim + 2 * g];
            wk[size_t(q) * ng * 2 + (g / 4) * 8 + g % 4] = lo;
            wk[size_t(q) * ng * 2 + (g / 4) * 8 + 4 + g % 4] = hi;
            wsum += lo + hi;
        }
        zeros[q] = -128 * wsum;                                              // search.rs:2842
    }
    if (n_threads < 1) n_threads = 1;
    const int64_t n_qb = (nq + 7) / 8;
    int64_t n_ranges = std::max<int64_t>(1, std::min<int64_t>(n_blocks / 64, (int64_t(n_threads) * 4 + n_qb - 1) / n_qb));
    const int64_t per_range = ((n_blocks + n_ranges - 1) / n_ranges + 1) / 2 * 2;
    n_ranges = (n_blocks + per_range - 1) / per_range;
    std::vector<std::vector<TopK>> heaps(n_ranges, std::vector<TopK>(nq, TopK(int(k))));
    std::vector<std::pair<int64_t, int64_t>> tiles;
    for (int64_t r = 0; r < n_ranges; ++r) for (int64_t qb = 0; qb < n_qb; ++qb) tiles.push_back({r, qb});   // range-major
    std::atomic<size_t> next{0};
    auto worker = [&]() {
        for (;;) {
            const size_t t = next.fetch_add(1);
            if (t >= tiles.size()) return;
            const int64_t r = tiles[t].first, q0 = tiles[t].second * 8;
            const int nqb = int(std::min<int64_t>(8, nq - q0));
            const int8_t *wp[8];
            for (int q = 0; q < nqb; ++q) wp[q] = wk.data() + size_t(q0 + q) * ng * 2;
            scan_tile(vm_codes, quads, vec_scales, n, r * per_range, std::min(n_blocks, (r + 1) * per_range), levels, wp,
                      zeros.data() + q0, qscale + q0, qbias + q0, nqb, mask, heaps[r].data() + q0);
        }
    };
    std::vector<std::thread> pool;
    for (int t = 1; t < n_threads; ++t) pool.emplace_back(worker);
    worker();
    for (auto &th : pool) th.join();
    for (int64_t q = 0; q < nq; ++q) {
        std::vector<Cand> all;
        for (int64_t r = 0; r < n_ranges; ++r) all.insert(all.end(), heaps[r][q].v.begin(), heaps[r][q].v.end());
        std::sort(all.begin(), all.end(), better);
        for (int64_t j = 0; j < k; ++j) {
            scores_out[q * k + j] = j < int64_t(all.size()) ? all[j].s : -INFINITY;
            slots_out[q * k + j] = j < int64_t(all.size()) ? all[j].i : 0;
        }
    }
    return k;
}

}  // extern "C"
