/*
 * CPU oracle for the turbovec encode-and-scan path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the
 * reference's normative scalar algorithms; it is what the CUDA path is
 * checked against.  Nothing in the shipped library links, imports or calls
 * it.  Each function cites the reference source it follows (paths are
 * relative to the reference project root).
 *
 * Parity status: the encode half (rotation, codebook, calibration, codes,
 * scales, packing) is pinned absolutely by the reference's frozen goldens
 * (turbovec/tests/rotation_determinism.rs:75-96,
 *  turbovec/tests/codebook_determinism.rs:91-98,
 *  turbovec/tests/encode_fingerprint.rs:83-92).  The search half has no
 * frozen scores or id lists in the reference ("parity unpinned" there): it is
 * anchored on the reference's call sites and property tests only.
 *
 * Third-party arithmetic restated here because the crates are not vendored
 * in the reference tree:
 *   rand_chacha =0.3.1  (ChaCha, 8 rounds, 64-bit counter, word stream)
 *   statrs      =0.17.1 (Beta cdf / pdf; any accurate regularised incomplete
 *                        beta reproduces the f32 codebook hashes)
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see Makefile).
 * -ffp-contract=off matters: the reference never fuses a multiply and an add
 * unless it writes an explicit fma.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <float.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define TVO_BLOCK 32
#define TVO_FLUSH_EVERY 256

/* ------------------------------------------------------------------ */
/* ChaCha8 word stream (rand_chacha 0.3.1: key = 32 seed bytes as 8 LE */
/* words, 64-bit block counter starting at 0, stream id 0, output      */
/* consumed word by word; next_u64 = two consecutive words, low first) */
/* ------------------------------------------------------------------ */
typedef struct {
    uint32_t key[8];
    uint64_t counter;
    uint32_t buf[16];
    int idx;
} tvo_chacha8;

static inline uint32_t rotl32(uint32_t x, int n) { return (x << n) | (x >> (32 - n)); }

#define TVO_QR(a, b, c, d)                      \
    do {                                        \
        a += b; d ^= a; d = rotl32(d, 16);      \
        c += d; b ^= c; b = rotl32(b, 12);      \
        a += b; d ^= a; d = rotl32(d, 8);       \
        c += d; b ^= c; b = rotl32(b, 7);       \
    } while (0)

static void tvo_chacha8_block(tvo_chacha8 *s) {
    uint32_t st[16] = {0x61707865u, 0x3320646eu, 0x79622d32u, 0x6b206574u};
    for (int i = 0; i < 8; i++) st[4 + i] = s->key[i];
    st[12] = (uint32_t)(s->counter & 0xffffffffu);
    st[13] = (uint32_t)(s->counter >> 32);
    st[14] = 0; st[15] = 0;
    uint32_t w[16];
    memcpy(w, st, sizeof w);
    for (int r = 0; r < 4; r++) {       /* 8 rounds = 4 double rounds */
        TVO_QR(w[0], w[4], w[8], w[12]);
        TVO_QR(w[1], w[5], w[9], w[13]);
        TVO_QR(w[2], w[6], w[10], w[14]);
        TVO_QR(w[3], w[7], w[11], w[15]);
        TVO_QR(w[0], w[5], w[10], w[15]);
        TVO_QR(w[1], w[6], w[11], w[12]);
        TVO_QR(w[2], w[7], w[8], w[13]);
        TVO_QR(w[3], w[4], w[9], w[14]);
    }
    for (int i = 0; i < 16; i++) s->buf[i] = w[i] + st[i];
    s->counter++;
    s->idx = 0;
}

static void tvo_chacha8_init(tvo_chacha8 *s, const uint8_t seed[32]) {
    for (int i = 0; i < 8; i++)
        s->key[i] = (uint32_t)seed[4 * i] | ((uint32_t)seed[4 * i + 1] << 8) |
                    ((uint32_t)seed[4 * i + 2] << 16) | ((uint32_t)seed[4 * i + 3] << 24);
    s->counter = 0;
    s->idx = 16;
}

static uint32_t tvo_next_u32(tvo_chacha8 *s) {
    if (s->idx >= 16) tvo_chacha8_block(s);
    return s->buf[s->idx++];
}

static uint64_t tvo_next_u64(tvo_chacha8 *s) {
    uint64_t lo = tvo_next_u32(s);
    uint64_t hi = tvo_next_u32(s);
    return (hi << 32) | lo;
}

/* turbovec/src/rotation.rs:82-85 */
static const uint8_t TVO_ROTATION_SEED[32] = {
    164, 143, 161, 123, 88, 50, 61, 10, 234, 184, 161, 204, 105, 1, 20, 184,
    43, 140, 200, 117, 24, 180, 247, 84, 141, 68, 110, 161, 228, 223, 32, 242};

/*
 * Rotation tables.  turbovec/src/rotation.rs:141-187 (Rotation::new) and
 * :990-997 (fisher_yates).  signs: 2*dim floats (+1/-1), perms: 2*dim u32;
 * perm[i] is the SOURCE coordinate of output slot i.
 */
void tvo_rotation_tables(int dim, float *signs, uint32_t *perms) {
    tvo_chacha8 rng;
    tvo_chacha8_init(&rng, TVO_ROTATION_SEED);
    for (int r = 0; r < 2; r++) {
        float *sg = signs + (size_t)r * dim;
        uint32_t *pm = perms + (size_t)r * dim;
        for (int i = 0; i < dim; i++) sg[i] = (tvo_next_u32(&rng) & 1u) ? -1.0f : 1.0f;
        for (int i = 0; i < dim; i++) pm[i] = (uint32_t)i;
        for (int i = dim - 1; i >= 1; i--) {
            uint64_t j = tvo_next_u64(&rng) % ((uint64_t)i + 1);
            uint32_t t = pm[i]; pm[i] = pm[j]; pm[j] = t;
        }
    }
}

int tvo_block_size(int dim) { return dim & (-dim); } /* rotation.rs:92-95 */

/* rotation.rs:964-982 (wht_block_scalar) */
static void tvo_wht_block(float *blk, int block, float inv_sqrt_block) {
    for (int len = 1; len < block; len <<= 1) {
        for (int i = 0; i < block; i += 2 * len) {
            for (int j = i; j < i + len; j++) {
                float a = blk[j], b = blk[j + len];
                blk[j] = a + b;
                blk[j + len] = a - b;
            }
        }
    }
    for (int i = 0; i < block; i++) blk[i] *= inv_sqrt_block;
}

/*
 * Rotate one row.  rotation.rs:218-256 (apply_scaled_into) computes
 * (src[perm0[i]]*inv)*sign0[i]; rotation.rs:265-320 (apply_with_scratch)
 * omits the inv multiply entirely.  use_inv selects between the two.
 * Round 1 multiplies by sign1 either at the gather or at the source slot
 * (signs1_pre); a multiply by +-1 is exact so both give the same bits.
 */
static void tvo_rotate_row(const float *src, int dim, const float *signs, const uint32_t *perms,
                           int use_inv, float inv, float *dst, float *scratch) {
    int block = tvo_block_size(dim);
    float inv_sqrt_block = 1.0f / sqrtf((float)block); /* rotation.rs:165 */
    const float *s0 = signs, *s1 = signs + dim;
    const uint32_t *p0 = perms, *p1 = perms + dim;
    for (int i = 0; i < dim; i++) {
        float v = src[p0[i]];
        scratch[i] = use_inv ? (v * inv) * s0[i] : v * s0[i];
    }
    for (int off = 0; off < dim; off += block) tvo_wht_block(scratch + off, block, inv_sqrt_block);
    for (int i = 0; i < dim; i++) dst[i] = scratch[p1[i]] * s1[i];
    for (int off = 0; off < dim; off += block) tvo_wht_block(dst + off, block, inv_sqrt_block);
}

/* Public: rotate nrows rows without normalisation (query path / goldens). */
void tvo_rotate_rows(const float *src, int nrows, int dim, float *dst) {
    float *signs = malloc(sizeof(float) * 2 * dim);
    uint32_t *perms = malloc(sizeof(uint32_t) * 2 * dim);
    float *scratch = malloc(sizeof(float) * dim);
    tvo_rotation_tables(dim, signs, perms);
    for (int r = 0; r < nrows; r++)
        tvo_rotate_row(src + (size_t)r * dim, dim, signs, perms, 0, 1.0f, dst + (size_t)r * dim, scratch);
    free(signs); free(perms); free(scratch);
}

/* ------------------------------------------------------------------ */
/* Beta(a,a) cdf / pdf and the Lloyd-Max codebook                      */
/* ------------------------------------------------------------------ */

/* Continued fraction for the incomplete beta function (modified Lentz). */
static double tvo_betacf(double a, double b, double x) {
    const double TINY = 1e-300, EPS = 1e-16;
    double qab = a + b, qap = a + 1.0, qam = a - 1.0;
    double c = 1.0, d = 1.0 - qab * x / qap;
    if (fabs(d) < TINY) d = TINY;
    d = 1.0 / d;
    double h = d;
    for (int m = 1; m <= 100000; m++) {
        double m2 = 2.0 * m;
        double aa = m * (b - m) * x / ((qam + m2) * (a + m2));
        d = 1.0 + aa * d; if (fabs(d) < TINY) d = TINY;
        c = 1.0 + aa / c; if (fabs(c) < TINY) c = TINY;
        d = 1.0 / d; h *= d * c;
        aa = -(a + m) * (qab + m) * x / ((a + m2) * (qap + m2));
        d = 1.0 + aa * d; if (fabs(d) < TINY) d = TINY;
        c = 1.0 + aa / c; if (fabs(c) < TINY) c = TINY;
        d = 1.0 / d;
        double del = d * c;
        h *= del;
        if (fabs(del - 1.0) < EPS) break;
    }
    return h;
}

/* Regularised incomplete beta I_x(a,b). */
double tvo_beta_cdf(double a, double b, double x) {
    if (x <= 0.0) return 0.0;
    if (x >= 1.0) return 1.0;
    double lbt = lgamma(a + b) - lgamma(a) - lgamma(b) + a * log(x) + b * log1p(-x);
    double bt = exp(lbt);
    if (x < (a + 1.0) / (a + b + 2.0)) return bt * tvo_betacf(a, b, x) / a;
    return 1.0 - bt * tvo_betacf(b, a, 1.0 - x) / b;
}

static double tvo_beta_pdf_sym(double a, double lnB, double t) {
    if (t <= 0.0 || t >= 1.0) return 0.0;
    return exp((a - 1.0) * log(t) + (a - 1.0) * log1p(-t) - lnB);
}

typedef struct { double a, lnB; } tvo_pdf_ctx;

static double tvo_integrand(const tvo_pdf_ctx *c, double x) {
    double t = (x + 1.0) / 2.0;                 /* codebook.rs:114-117 */
    return x * tvo_beta_pdf_sym(c->a, c->lnB, t) / 2.0;
}

/* codebook.rs:225-249 (adaptive_simpson_rec) */
static double tvo_simpson_rec(const tvo_pdf_ctx *c, double a, double b, double fa, double fb,
                              double fm, double whole, double tol, int depth) {
    double mid = (a + b) / 2.0, m1 = (a + mid) / 2.0, m2 = (mid + b) / 2.0;
    double fm1 = tvo_integrand(c, m1), fm2 = tvo_integrand(c, m2);
    double left = (mid - a) / 6.0 * (fa + 4.0 * fm1 + fm);
    double right = (b - mid) / 6.0 * (fm + 4.0 * fm2 + fb);
    double refined = left + right;
    if (depth == 0 || fabs(refined - whole) < 15.0 * tol) return refined + (refined - whole) / 15.0;
    return tvo_simpson_rec(c, a, mid, fa, fm, fm1, left, tol / 2.0, depth - 1) +
           tvo_simpson_rec(c, mid, b, fm, fb, fm2, right, tol / 2.0, depth - 1);
}

/* codebook.rs:214-223 (adaptive_simpson) */
static double tvo_simpson(const tvo_pdf_ctx *c, double a, double b, double tol, int depth) {
    double mid = (a + b) / 2.0;
    double fa = tvo_integrand(c, a), fb = tvo_integrand(c, b), fm = tvo_integrand(c, mid);
    double whole = (b - a) / 6.0 * (fa + 4.0 * fm + fb);
    return tvo_simpson_rec(c, a, b, fa, fb, fm, whole, tol, depth);
}

/*
 * Lloyd-Max codebook.  codebook.rs:69-167.  boundaries: 2^bits-1 floats,
 * centroids: 2^bits floats.
 */
void tvo_codebook(int bits, int dim, float *boundaries, float *centroids) {
    double a = ((double)dim - 1.0) / 2.0;
    tvo_pdf_ctx ctx = {a, 2.0 * lgamma(a) - lgamma(2.0 * a)};
    int n = 1 << bits;
    double std_dev = sqrt(2.0 * a / ((2.0 * a + 1.0) * 4.0 * a));
    double spread = 3.0 * std_dev;
    double c[16], nc[16], edges[17];
    for (int i = 0; i < n; i++) c[i] = -spread + 2.0 * spread * (double)i / ((double)n - 1.0);
    for (int it = 0; it < 200; it++) {
        edges[0] = -1.0;
        for (int i = 0; i < n - 1; i++) edges[i + 1] = (c[i] + c[i + 1]) / 2.0;
        edges[n] = 1.0;
        for (int i = 0; i < n; i++) {
            double lo = edges[i], hi = edges[i + 1];
            double prob = tvo_beta_cdf(a, a, (hi + 1.0) / 2.0) - tvo_beta_cdf(a, a, (lo + 1.0) / 2.0);
            if (prob < 1e-15) nc[i] = c[i];
            else nc[i] = tvo_simpson(&ctx, lo, hi, 1e-14, 50) / prob;
        }
        double max_change = 0.0;
        for (int i = 0; i < n; i++) {
            double d = fabs(c[i] - nc[i]);
            if (d > max_change) max_change = d;
            c[i] = nc[i];
        }
        if (max_change < 1e-12) break;
    }
    for (int i = 0; i < n; i++) centroids[i] = (float)c[i];
    for (int i = 0; i < n - 1; i++) boundaries[i] = (centroids[i] + centroids[i + 1]) * 0.5f;
}

/* ------------------------------------------------------------------ */
/* Encode                                                              */
/* ------------------------------------------------------------------ */

/* encode.rs:920-932 (norm_sq_scalar + combine_norm_chains) then sqrt (:900-916) */
float tvo_norm(const float *row, int dim) {
    float c[8] = {0};
    for (int j = 0; j < dim; j++) {
        float p = row[j] * row[j];
        c[j % 8] = c[j % 8] + p;
    }
    float s = ((c[0] + c[1]) + (c[2] + c[3])) + ((c[4] + c[5]) + (c[6] + c[7]));
    return sqrtf(s);
}

/* encode.rs:58-74: first flat index with !(|x| < 1e16), or -1. */
int64_t tvo_first_invalid(const float *x, int64_t len) {
    for (int64_t i = 0; i < len; i++)
        if (!(fabsf(x[i]) < 1e16f)) return i;
    return -1;
}

/*
 * Rotate a batch with 1/||row|| fused into the first gather.
 * encode.rs:406-458 (rotate_batch_into); zero-norm rule :446.
 */
void tvo_rotate_batch(const float *vectors, int64_t n, int dim, float *rotated, float *norms) {
    float *signs = malloc(sizeof(float) * 2 * dim);
    uint32_t *perms = malloc(sizeof(uint32_t) * 2 * dim);
    tvo_rotation_tables(dim, signs, perms);
#pragma omp parallel
    {
        float *scratch = malloc(sizeof(float) * dim);
#pragma omp for schedule(static)
        for (int64_t i = 0; i < n; i++) {
            const float *src = vectors + (size_t)i * dim;
            float nv = tvo_norm(src, dim);
            norms[i] = nv;
            float inv = nv > 1e-10f ? 1.0f / nv : 0.0f;
            tvo_rotate_row(src, dim, signs, perms, 1, inv, rotated + (size_t)i * dim, scratch);
        }
        free(scratch);
    }
    free(signs); free(perms);
}

static int tvo_cmp_f32(const void *a, const void *b) {
    float x = *(const float *)a, y = *(const float *)b;
    return (x > y) - (x < y);
}

/*
 * TQ+ calibration fit on already-rotated rows.
 * encode.rs:364-369 (tqplus_anchor), :737-857 (compute_tqplus_calibration).
 * The reference selects two order statistics per coordinate with
 * select_nth_unstable on total-order keys; a full sort yields the same two
 * values.
 */
void tvo_fit_calibration(const float *rotated, int64_t n, int dim, const float *centroids,
                         int n_centroids, float *shift, float *scale) {
    double a = ((double)dim - 1.0) / 2.0;
    float c_outer = 0.0f;
    for (int i = 0; i < n_centroids; i++) {
        float v = fabsf(centroids[i]);
        if (v > c_outer) c_outer = v;
    }
    double p_hi = tvo_beta_cdf(a, a, ((double)c_outer + 1.0) / 2.0);
    double p_lo = 1.0 - p_hi;
    float qc_lo = -c_outer, qc_hi = c_outer;
    float qc_span = qc_hi - qc_lo;
    int64_t lo_idx = (int64_t)((double)n * p_lo);
    int64_t hi_idx = (int64_t)((double)n * p_hi);
    if (hi_idx > n - 1) hi_idx = n - 1;
    if (hi_idx < lo_idx + 1) hi_idx = lo_idx + 1;
    float *col = malloc(sizeof(float) * n);
    for (int d = 0; d < dim; d++) {
        shift[d] = 0.0f; scale[d] = 1.0f;
        for (int64_t i = 0; i < n; i++) col[i] = rotated[(size_t)i * dim + d];
        qsort(col, n, sizeof(float), tvo_cmp_f32);
        float qe_lo = col[lo_idx], qe_hi = col[hi_idx];
        float qe_span = qe_hi - qe_lo;
        if (qe_span > 1e-6f) {
            scale[d] = qc_span / qe_span;
            shift[d] = qc_lo / scale[d] - qe_lo;
        }
    }
    free(col);
}

/*
 * Quantise + scale one rotated row.  encode.rs:1418-1476
 * (fused_quantize_scale_pack_scalar), :276-278 (recon_entry),
 * :1194-1200 (scale_from_inner).  codes_out receives one code per coordinate.
 * shift/scale_tq may be NULL (identity pair, encode.rs:578-589).
 */
static float tvo_quantize_row(const float *rot, int dim, int bits, const float *boundaries,
                              const float *centroids, const float *shift, const float *scale_tq,
                              float norm, uint8_t *codes_out) {
    double chains[4] = {0, 0, 0, 0};
    int nb = (1 << bits) - 1;
    for (int j = 0; j < dim; j++) {
        float sh = shift ? shift[j] : 0.0f;
        float sc = scale_tq ? scale_tq[j] : 1.0f;
        float inv_sc = 1.0f / sc;                      /* encode.rs:593 */
        float calib = (rot[j] + sh) * sc;
        uint8_t v = 0;
        for (int bi = 0; bi < nb; bi++)
            if (calib > boundaries[bi]) v++;
        codes_out[j] = v;
        double recon = (double)centroids[v] * (double)inv_sc - (double)sh;
        double term = (double)rot[j] * recon;
        chains[j % 4] = chains[j % 4] + term;
    }
    double inner = (chains[0] + chains[1]) + (chains[2] + chains[3]);
    if (inner > 0.1) return norm / (float)inner;
    return 0.0f;
}

/* Bit-plane packing of one row.  encode.rs:1464-1470. */
static void tvo_pack_bitplane_row(const uint8_t *codes, int dim, int bits, uint8_t *packed_row) {
    int bpp = dim / 8;
    for (int c = 0; c < bpp; c++)
        for (int p = 0; p < bits; p++) {
            uint8_t byte = 0;
            for (int k = 0; k < 8; k++) byte |= (uint8_t)(((codes[8 * c + k] >> p) & 1) << (7 - k));
            packed_row[p * bpp + c] = byte;
        }
}

/*
 * Full encode of a batch: encode.rs:510-541 (encode) + :560-652.
 * packed_out: n * bits*dim/8 bytes (bit-plane rows); scales_out: n floats;
 * codes_out (optional): n*dim per-coordinate codes; rotated_out (optional).
 */
void tvo_encode(const float *vectors, int64_t n, int dim, int bits, const float *boundaries,
                const float *centroids, const float *shift, const float *scale_tq,
                uint8_t *packed_out, float *scales_out, uint8_t *codes_out, float *rotated_out) {
    float *rotated = rotated_out ? rotated_out : malloc(sizeof(float) * (size_t)n * dim);
    float *norms = malloc(sizeof(float) * (n > 0 ? n : 1));
    tvo_rotate_batch(vectors, n, dim, rotated, norms);
    int bytes_per_row = bits * dim / 8;
#pragma omp parallel
    {
        uint8_t *codes = malloc(dim);
#pragma omp for schedule(static)
        for (int64_t i = 0; i < n; i++) {
            scales_out[i] = tvo_quantize_row(rotated + (size_t)i * dim, dim, bits, boundaries, centroids,
                                             shift, scale_tq, norms[i], codes);
            if (packed_out) tvo_pack_bitplane_row(codes, dim, bits, packed_out + (size_t)i * bytes_per_row);
            if (codes_out) memcpy(codes_out + (size_t)i * dim, codes, dim);
        }
        free(codes);
    }
    free(norms);
    if (!rotated_out) free(rotated);
}

/*
 * Re-encoding of stored rows under a new TQ+ pair: lib.rs:2760-2832 (reencode_stored_rows).
 * Each row is reconstructed from its codes under the committed pair (NULL = identity),
 * x[d] = centroids[code] * old_inv[d] - old_shift[d] in f32, its squared length is summed in one
 * f64 chain in coordinate order, the effective norm is (f64(scale_old) * sumsq) as f32, and the
 * reconstruction goes through the same quantise + scale as a fresh row under the new pair.
 * codes_in / codes_out: one code per coordinate, n * dim.
 */
void tvo_reencode(const uint8_t *codes_in, const float *scales_in, int64_t n, int dim, int bits,
                  const float *boundaries, const float *centroids, const float *old_shift,
                  const float *old_scale, const float *new_shift, const float *new_scale,
                  uint8_t *codes_out, float *scales_out) {
#pragma omp parallel
    {
        float *recon = malloc(sizeof(float) * dim);
#pragma omp for schedule(static)
        for (int64_t i = 0; i < n; i++) {
            double sumsq = 0.0;
            for (int d = 0; d < dim; d++) {
                float inv = old_scale ? 1.0f / old_scale[d] : 1.0f;
                float sh = old_shift ? old_shift[d] : 0.0f;
                float x = centroids[codes_in[(size_t)i * dim + d]] * inv - sh;
                recon[d] = x;
                sumsq += (double)x * (double)x;
            }
            float norm = (float)((double)scales_in[i] * sumsq);
            scales_out[i] = tvo_quantize_row(recon, dim, bits, boundaries, centroids, new_shift, new_scale,
                                             norm, codes_out + (size_t)i * dim);
        }
        free(recon);
    }
}

/*
 * Per-coordinate distance to the nearest quantiser decision boundary, for the
 * classification of code mismatches (a mismatch is tolerated only within
 * 1e-6 of a boundary).  Same calib expression as tvo_quantize_row.
 */
void tvo_boundary_distance(const float *rotated, int64_t n, int dim, int bits, const float *boundaries,
                           const float *shift, const float *scale_tq, float *dist_out) {
    int nb = (1 << bits) - 1;
    for (int64_t i = 0; i < n; i++)
        for (int j = 0; j < dim; j++) {
            float sh = shift ? shift[j] : 0.0f, sc = scale_tq ? scale_tq[j] : 1.0f;
            float calib = (rotated[(size_t)i * dim + j] + sh) * sc;
            float best = FLT_MAX;
            for (int bi = 0; bi < nb; bi++) {
                float d = fabsf(calib - boundaries[bi]);
                if (d < best) best = d;
            }
            dist_out[(size_t)i * dim + j] = best;
        }
}

/* ------------------------------------------------------------------ */
/* Layouts (pack.rs)                                                   */
/* ------------------------------------------------------------------ */

int tvo_ngroups(int dim, int bits) { return dim / (8 / bits); } /* pack.rs:252-257 */

/*
 * Bit-plane rows -> byte-group codes.  pack.rs:264-334: coordinate
 * g*cpb + k sits at shift (cpb-1-k)*field, field = 4 for 3-bit.
 */
void tvo_extract_codes_flat(const uint8_t *packed, int64_t n, int bits, int dim, uint8_t *flat) {
    int bpp = dim / 8, cpb = 8 / bits, ng = dim / cpb, bpr = bits * bpp;
    int field = bits == 3 ? 4 : bits;
    memset(flat, 0, (size_t)n * ng);
    for (int64_t v = 0; v < n; v++)
        for (int j = 0; j < dim; j++) {
            int c = j / 8, k = j % 8, code = 0;
            for (int p = 0; p < bits; p++)
                code |= ((packed[(size_t)v * bpr + p * bpp + c] >> (7 - k)) & 1) << p;
            int g = j / cpb;
            int sh = (cpb - 1 - (j % cpb)) * field;
            flat[(size_t)v * ng + g] |= (uint8_t)(code << sh);
        }
}

/* pack.rs:340-361 (pack_blocked_sequential): (block*ng + g)*32 + lane, zero padding. */
void tvo_pack_blocked_seq(const uint8_t *flat, int64_t n, int ng, uint8_t *blocked) {
    int64_t n_blocks = (n + TVO_BLOCK - 1) / TVO_BLOCK;
    memset(blocked, 0, (size_t)n_blocks * ng * TVO_BLOCK);
    for (int64_t v = 0; v < n; v++) {
        int64_t b = v / TVO_BLOCK; int lane = (int)(v % TVO_BLOCK);
        for (int g = 0; g < ng; g++) blocked[((size_t)b * ng + g) * TVO_BLOCK + lane] = flat[(size_t)v * ng + g];
    }
}

/* pack.rs:375-467 (seq_to_packed): blocked bytes -> bit-plane rows. */
void tvo_seq_to_packed(const uint8_t *blocked, int64_t n, int bits, int dim, uint8_t *packed) {
    int bpp = dim / 8, cpb = 8 / bits, ng = dim / cpb, bpr = bits * bpp;
    int field = bits == 3 ? 4 : bits;
    memset(packed, 0, (size_t)n * bpr);
    for (int64_t v = 0; v < n; v++) {
        int64_t b = v / TVO_BLOCK; int lane = (int)(v % TVO_BLOCK);
        for (int j = 0; j < dim; j++) {
            int g = j / cpb, sh = (cpb - 1 - (j % cpb)) * field;
            int code = (blocked[((size_t)b * ng + g) * TVO_BLOCK + lane] >> sh) & ((1 << bits) - 1);
            int c = j / 8, k = j % 8;
            for (int p = 0; p < bits; p++)
                packed[(size_t)v * bpr + p * bpp + c] |= (uint8_t)(((code >> p) & 1) << (7 - k));
        }
    }
}

/* ------------------------------------------------------------------ */
/* Search                                                              */
/* ------------------------------------------------------------------ */

enum {
    TVO_MODE_AUTO = 0,        /* what an AVX-512 VBMI+VNNI x86 host selects */
    TVO_MODE_PD = 1,          /* permute-dot int8 (4-bit, ngroups % 4 == 0)  */
    TVO_MODE_LUT_MULADD = 2,  /* u8 LUT, (f32)isum*scale + bias  (search.rs:1176) */
    TVO_MODE_LUT_FLUSH = 3,   /* u8 LUT, fma per 256-group batch (search.rs:1596) */
    TVO_MODE_LUT_SCALAR = 4   /* u8 LUT, score += scale*u8 per lookup (search.rs:3125) */
};

/*
 * Kernel-family selection.  pack.rs:1260-1263 (vector_major_for),
 * search.rs:2975-2980 (pd iff vm && bits == 4), dispatch search.rs:4089-4216.
 */
int tvo_resolve_mode(int mode, int bits, int ngroups) {
    if (mode != TVO_MODE_AUTO) return mode;
    int vm = (ngroups % 4) == 0;
    if (vm && bits == 4) return TVO_MODE_PD;
    if (vm) return TVO_MODE_LUT_MULADD;
    return TVO_MODE_LUT_FLUSH;
}

/* Rust f32::round: half away from zero == C roundf. */

/*
 * u8 lookup tables for one query.  search.rs:2856-2994
 * (build_query_neon_lut_from_slice).  luts: ngroups*32 bytes, first 16 of a
 * group indexed by byte>>4 (earlier coordinates), next 16 by byte&15.
 */
void tvo_build_lut(const float *q, const float *centroids, int bits, int dim, uint8_t *luts,
                   float *scale_out, float *bias_out) {
    int cpb = 8 / bits, cpn = cpb / 2, ng = dim / cpb;
    unsigned code_mask = (1u << bits) - 1;
    float *fv = malloc(sizeof(float) * (size_t)ng * 32);
    float *mins = malloc(sizeof(float) * (size_t)ng * 2);
    float max_span = 0.0f, bias = 0.0f;
    for (int g = 0; g < ng; g++) {
        int d0 = g * cpb;
        float mn[2], mx[2];
        for (int half = 0; half < 2; half++) {
            float lo_min = FLT_MAX, lo_max = -FLT_MAX;
            for (unsigned nib = 0; nib < 16; nib++) {
                float s = 0.0f;
                for (int c = 0; c < cpn; c++) {
                    int sh = (cpn - 1 - c) * bits;
                    unsigned code = (nib >> sh) & code_mask;
                    float p = q[d0 + half * cpn + c] * centroids[code];
                    s = s + p;
                }
                fv[g * 32 + half * 16 + nib] = s;
                if (s < lo_min) lo_min = s;
                if (s > lo_max) lo_max = s;
            }
            mn[half] = lo_min; mx[half] = lo_max;
        }
        mins[g * 2] = mn[0]; mins[g * 2 + 1] = mn[1];
        float pair = mn[0] + mn[1];
        bias = bias + pair;
        float s0 = mx[0] - mn[0], s1 = mx[1] - mn[1];
        if (s0 > max_span) max_span = s0;
        if (s1 > max_span) max_span = s1;
    }
    float scale = max_span > 0.0f ? max_span / 127.0f : 1.0f;
    float inv_scale;
    if (scale >= FLT_MIN) inv_scale = 1.0f / scale;
    else { scale = 1.0f; inv_scale = 1.0f; }
    for (int g = 0; g < ng; g++)
        for (int half = 0; half < 2; half++)
            for (int i = 0; i < 16; i++) {
                int j = g * 32 + half * 16 + i;
                float r = roundf((fv[j] - mins[g * 2 + half]) * inv_scale);
                if (r < 0.0f) r = 0.0f;
                if (r > 127.0f) r = 127.0f;
                luts[j] = (uint8_t)r;
            }
    *scale_out = scale; *bias_out = bias;
    free(fv); free(mins);
}

static int8_t tvo_round_clamp_i8(float v) {
    float r = roundf(v);
    if (r < -127.0f) r = -127.0f;
    if (r > 127.0f) r = 127.0f;
    return (int8_t)r;
}

/*
 * Permute-dot tables for one query.  search.rs:2806-2846 (build_permute_dot).
 * weights are returned in plain coordinate order (w[d]); the reference's
 * storage order (lo/hi quads) is a kernel detail that does not change sums.
 */
void tvo_build_pd(const float *q, const float *centroids, int dim, int8_t *levels, int8_t *weights,
                  float *scale_out) {
    float cmax = 0.0f;
    for (int i = 0; i < 16; i++) { float v = fabsf(centroids[i]); if (v > cmax) cmax = v; }
    float cs = cmax > 0.0f ? cmax / 127.0f : 1.0f;
    for (int i = 0; i < 16; i++) levels[i] = tvo_round_clamp_i8(centroids[i] / cs);
    float qmax = 0.0f;
    for (int d = 0; d < dim; d++) { float v = fabsf(q[d]); if (v > qmax) qmax = v; }
    float qs = qmax / 127.0f, inv_qs;
    if (qs >= FLT_MIN) inv_qs = 1.0f / qs;
    else { qs = 1.0f; inv_qs = 1.0f; }
    for (int d = 0; d < dim; d++) weights[d] = tvo_round_clamp_i8(q[d] * inv_qs);
    *scale_out = cs * qs;
}

/* Total order of results: score descending, slot ascending (search.rs:236-252, 4285-4290). */
static inline int tvo_better(float s, int64_t i, float s2, int64_t i2) {
    return s > s2 || (s == s2 && i < i2);
}

typedef struct { float *s; int64_t *i; int sz, k; } tvo_topk;

static void tvo_topk_push(tvo_topk *h, float s, int64_t idx) {
    if (h->sz == h->k) {
        if (!tvo_better(s, idx, h->s[h->k - 1], h->i[h->k - 1])) return;
        h->sz--;
    }
    int p = h->sz++;
    while (p > 0 && tvo_better(s, idx, h->s[p - 1], h->i[p - 1])) {
        h->s[p] = h->s[p - 1]; h->i[p] = h->i[p - 1]; p--;
    }
    h->s[p] = s; h->i[p] = idx;
}

/* search.rs:3000-3004 */
static inline int tvo_mask_allows(const uint64_t *mask, int64_t slot) {
    return (int)((mask[slot >> 6] >> (slot & 63)) & 1);
}

/*
 * Search.  search.rs:3206-4353 with the block scan written in the scalar
 * form of search.rs:3077-3147; integer sums are exact in every reference
 * kernel, so only the float epilogue differs per mode (see the enum).
 *
 * blocked: sequential-blocked codes; mask: little-endian u64 words or NULL;
 * shift/scale_tq NULL when uncalibrated.  Outputs nq*k_eff entries, row
 * major; returns k_eff = min(k, n_allowed).
 */
int64_t tvo_search(const float *queries, int64_t nq, int dim, int bits, const uint8_t *blocked,
                   const float *vec_scales, int64_t n, const float *centroids, const float *shift,
                   const float *scale_tq, int64_t k, const uint64_t *mask, int mode,
                   float *scores_out, int64_t *slots_out) {
    int64_t n_allowed = n;
    if (mask) {
        n_allowed = 0;
        for (int64_t w = 0; w < (n + 63) / 64; w++) n_allowed += __builtin_popcountll(mask[w]);
    }
    if (k > n_allowed) k = n_allowed;
    if (k <= 0 || nq <= 0) return k < 0 ? 0 : k;
    int cpb = 8 / bits, ng = dim / cpb;
    mode = tvo_resolve_mode(mode, bits, ng);
    int64_t n_blocks = (n + TVO_BLOCK - 1) / TVO_BLOCK;

    /* query preparation: rotate (no normalisation), TQ+ inverse, tables */
    float *q_rot = malloc(sizeof(float) * (size_t)nq * dim);
    tvo_rotate_rows(queries, (int)nq, dim, q_rot);
    float *bias_corr = calloc(nq, sizeof(float));
    if (shift) {                                      /* search.rs:3154-3186 */
        for (int64_t qi = 0; qi < nq; qi++) {
            double bc = 0.0;
            float *row = q_rot + (size_t)qi * dim;
            for (int d = 0; d < dim; d++) {
                bc = bc - (double)row[d] * (double)shift[d];
                row[d] = row[d] / scale_tq[d];
            }
            bias_corr[qi] = (float)bc;
        }
    }
    uint8_t *luts = NULL; int8_t *weights = NULL; int8_t levels[16];
    float *qscale = malloc(sizeof(float) * nq), *qbias = malloc(sizeof(float) * nq);
    if (mode == TVO_MODE_PD) {
        weights = malloc((size_t)nq * dim);
        for (int64_t qi = 0; qi < nq; qi++) {
            tvo_build_pd(q_rot + (size_t)qi * dim, centroids, dim, levels, weights + (size_t)qi * dim, &qscale[qi]);
            qbias[qi] = 0.0f + bias_corr[qi];          /* search.rs:2844, 3262-3266 */
        }
    } else {
        luts = malloc((size_t)nq * ng * 32);
        for (int64_t qi = 0; qi < nq; qi++) {
            float b;
            tvo_build_lut(q_rot + (size_t)qi * dim, centroids, bits, dim, luts + (size_t)qi * ng * 32, &qscale[qi], &b);
            qbias[qi] = b + bias_corr[qi];             /* search.rs:3260 */
        }
    }

    int nthreads = 1;
#ifdef _OPENMP
    nthreads = omp_get_max_threads();
#endif
    float *hs = malloc(sizeof(float) * (size_t)nthreads * nq * k);
    int64_t *hi = malloc(sizeof(int64_t) * (size_t)nthreads * nq * k);
    int *hsz = calloc((size_t)nthreads * nq, sizeof(int));

#pragma omp parallel
    {
        int tid = 0;
#ifdef _OPENMP
        tid = omp_get_thread_num();
#endif
        int8_t *lev_tile = (mode == TVO_MODE_PD) ? malloc((size_t)TVO_BLOCK * dim) : NULL;
#pragma omp for schedule(static)
        for (int64_t b = 0; b < n_blocks; b++) {
            int64_t base = b * TVO_BLOCK;
            if (mask) {                                 /* search.rs:3015-3029 */
                uint64_t word = mask[base >> 6];
                if (((word >> (base & 63)) & 0xFFFFFFFFull) == 0) continue;
            }
            const uint8_t *blk = blocked + (size_t)b * ng * TVO_BLOCK;
            int lanes = (int)((n - base) < TVO_BLOCK ? (n - base) : TVO_BLOCK);
            if (mode == TVO_MODE_PD) {
                /* high nibble = even coordinate, low nibble = odd (search.rs:2787-2790) */
                for (int g = 0; g < ng; g++)
                    for (int l = 0; l < lanes; l++) {
                        uint8_t byte = blk[g * TVO_BLOCK + l];
                        lev_tile[(size_t)l * dim + 2 * g] = levels[byte >> 4];
                        lev_tile[(size_t)l * dim + 2 * g + 1] = levels[byte & 15];
                    }
            }
            for (int64_t qi = 0; qi < nq; qi++) {
                tvo_topk h = {hs + ((size_t)tid * nq + qi) * k, hi + ((size_t)tid * nq + qi) * k,
                              hsz[(size_t)tid * nq + qi], (int)k};
                const uint8_t *lut = luts ? luts + (size_t)qi * ng * 32 : NULL;
                const int8_t *w = weights ? weights + (size_t)qi * dim : NULL;
                float sc = qscale[qi], bi = qbias[qi];
                for (int l = 0; l < lanes; l++) {
                    int64_t vi = base + l;
                    if (mask && !tvo_mask_allows(mask, vi)) continue;
                    float score;
                    if (mode == TVO_MODE_PD) {
                        int32_t isum = 0;
                        const int8_t *lv = lev_tile + (size_t)l * dim;
                        for (int d = 0; d < dim; d++) isum += (int32_t)w[d] * (int32_t)lv[d];
                        score = fmaf((float)isum, sc, bi);            /* search.rs:1523 */
                    } else if (mode == TVO_MODE_LUT_MULADD) {
                        uint32_t isum = 0;
                        for (int g = 0; g < ng; g++) {
                            uint8_t byte = blk[g * TVO_BLOCK + l];
                            isum += lut[g * 32 + (byte >> 4)] + lut[g * 32 + 16 + (byte & 15)];
                        }
                        float t = (float)(int32_t)isum * sc;
                        score = t + bi;                               /* search.rs:1176 */
                    } else if (mode == TVO_MODE_LUT_FLUSH) {
                        float acc = bi;
                        for (int g0 = 0; g0 < ng; g0 += TVO_FLUSH_EVERY) {
                            int g1 = g0 + TVO_FLUSH_EVERY < ng ? g0 + TVO_FLUSH_EVERY : ng;
                            uint32_t isum = 0;
                            for (int g = g0; g < g1; g++) {
                                uint8_t byte = blk[g * TVO_BLOCK + l];
                                isum += lut[g * 32 + (byte >> 4)] + lut[g * 32 + 16 + (byte & 15)];
                            }
                            acc = fmaf(sc, (float)(int32_t)isum, acc); /* search.rs:1596 */
                        }
                        score = acc;
                    } else {
                        score = bi;                                   /* search.rs:3115-3127 */
                        for (int g = 0; g < ng; g++) {
                            uint8_t byte = blk[g * TVO_BLOCK + l];
                            float t0 = sc * (float)lut[g * 32 + (byte >> 4)];
                            score = score + t0;
                            float t1 = sc * (float)lut[g * 32 + 16 + (byte & 15)];
                            score = score + t1;
                        }
                    }
                    score = score * vec_scales[vi];
                    tvo_topk_push(&h, score, vi);
                }
                hsz[(size_t)tid * nq + qi] = h.sz;
            }
        }
        free(lev_tile);
    }

    /* merge per-thread lists: sort by (score desc, slot asc), truncate k (search.rs:4285-4298) */
    for (int64_t qi = 0; qi < nq; qi++) {
        float *ms = scores_out + (size_t)qi * k;
        int64_t *mi = slots_out + (size_t)qi * k;
        tvo_topk h = {ms, mi, 0, (int)k};
        for (int t = 0; t < nthreads; t++) {
            int sz = hsz[(size_t)t * nq + qi];
            for (int e = 0; e < sz; e++)
                tvo_topk_push(&h, hs[((size_t)t * nq + qi) * k + e], hi[((size_t)t * nq + qi) * k + e]);
        }
        for (int e = h.sz; e < k; e++) { ms[e] = -INFINITY; mi[e] = 0; } /* search.rs:4341-4352 */
    }
    free(q_rot); free(bias_corr); free(luts); free(weights); free(qscale); free(qbias);
    free(hs); free(hi); free(hsz);
    return k;
}

/* Query-table access for tests that compare the device query preparation. */
void tvo_query_tables(const float *queries, int64_t nq, int dim, int bits, const float *centroids,
                      const float *shift, const float *scale_tq, int mode, float *q_rot_out,
                      uint8_t *luts_out, int8_t *weights_out, int8_t *levels_out, float *scale_out,
                      float *bias_out) {
    int ng = dim / (8 / bits);
    mode = tvo_resolve_mode(mode, bits, ng);
    tvo_rotate_rows(queries, (int)nq, dim, q_rot_out);
    for (int64_t qi = 0; qi < nq; qi++) {
        float *row = q_rot_out + (size_t)qi * dim;
        float corr = 0.0f;
        if (shift) {
            double bc = 0.0;
            for (int d = 0; d < dim; d++) {
                bc = bc - (double)row[d] * (double)shift[d];
                row[d] = row[d] / scale_tq[d];
            }
            corr = (float)bc;
        }
        if (mode == TVO_MODE_PD) {
            tvo_build_pd(row, centroids, dim, levels_out, weights_out + (size_t)qi * dim, &scale_out[qi]);
            bias_out[qi] = 0.0f + corr;
        } else {
            float b;
            tvo_build_lut(row, centroids, bits, dim, luts_out + (size_t)qi * ng * 32, &scale_out[qi], &b);
            bias_out[qi] = b + corr;
        }
    }
}

/* FNV-1a 64 over bytes (turbovec/tests/common/fingerprint.rs:59-66). */
uint64_t tvo_fnv1a(const uint8_t *bytes, int64_t len) {
    uint64_t h = 0xcbf29ce484222325ull;
    for (int64_t i = 0; i < len; i++) { h ^= bytes[i]; h *= 0x100000001b3ull; }
    return h;
}

/* LCG fixture vectors (turbovec/tests/common/fingerprint.rs:80-96). */
void tvo_lcg_vectors(int64_t count, uint64_t seed, float *out) {
    uint64_t state = seed | 1;
    for (int64_t i = 0; i < count; i++) {
        state = state * 6364136223846793005ull + 1442695040888963407ull;
        out[i] = (float)((double)(uint32_t)(state >> 32) / 2147483648.0 - 1.0);
    }
}
