/*
 * CPU oracle for the tachyon decode / prefill hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference engine (juliog922/tachyon) for the
 * batch-1 decode step: the quantised layouts, the matrix-vector product, RMS-norm, RoPE, GeGLU, decode
 * attention over a ring cache, the greedy sampler and the whole Gemma-4-style decoder forward pass.  It
 * exists so that the CUDA kernels can be compared against an independent scalar implementation on the
 * same seeded inputs; it is linked only by the tests, the smoke check and the benchmark's CPU-baseline
 * legs.  Nothing in the shipped library calls it and it is not a fallback.
 *
 * Every function cites the reference file and lines it follows (paths relative to the reference root).
 * Parity status: the format code (f16 conversion, Q4 packing, Q8 block quantisation) is pinned by the
 * reference's own known-answer tests (crates/tachyon/src/quant.rs:249-277), which tests/ re-run against
 * this file.  The decoder forward restates crates/tachyon/tests/common/tiny.rs:225-386; the reference
 * ships no golden outputs for it that can be used without its real checkpoints.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <unistd.h>

#define TBO_API __attribute__((visibility("default")))

/* A minimal parallel-for over [0, n) on POSIX threads (this image's gcc has no OpenMP runtime). */
static int g_threads = 0;
typedef void (*range_fn)(void *ctx, long lo, long hi);
typedef struct { range_fn fn; void *ctx; long lo, hi; } range_job;
static void *range_main(void *p) { range_job *j = (range_job *)p; j->fn(j->ctx, j->lo, j->hi); return NULL; }
static int threads_now(void) {
    if (g_threads <= 0) { long n = sysconf(_SC_NPROCESSORS_ONLN); g_threads = n > 0 ? (int)(n > 256 ? 256 : n) : 1; }
    return g_threads;
}
static void parallel_for(long n, long grain, range_fn fn, void *ctx) {
    int t = threads_now();
    if (n / (grain > 0 ? grain : 1) < t) t = (int)(n / (grain > 0 ? grain : 1));
    if (t <= 1) { fn(ctx, 0, n); return; }
    pthread_t th[256];
    range_job jobs[256];
    for (int i = 0; i < t; i++) {
        jobs[i].fn = fn; jobs[i].ctx = ctx; jobs[i].lo = n * i / t; jobs[i].hi = n * (i + 1) / t;
        if (i + 1 < t) pthread_create(&th[i], NULL, range_main, &jobs[i]);
    }
    range_main(&jobs[t - 1]);
    for (int i = 0; i + 1 < t; i++) pthread_join(th[i], NULL);
}

/* ------------------------------------------------------------------------------------------------ */
/* f16 <-> f32, exact.  crates/tachyon/src/quant.rs:133-158                                          */
/* ------------------------------------------------------------------------------------------------ */

static uint32_t round_kept(uint32_t kept, uint32_t shift, uint32_t bits) {
    uint32_t rem = bits & ((1u << shift) - 1u), half = 1u << (shift - 1u);
    return kept + ((rem > half || (rem == half && (kept & 1u))) ? 1u : 0u);
}

TBO_API uint16_t tbo_f16_bits(float v) {
    uint32_t b;
    memcpy(&b, &v, 4);
    uint32_t sign = (b >> 16) & 0x8000u, man = b & 0x7fffffu;
    int exp = (int)((b >> 23) & 0xffu), e = exp - 112;
    uint32_t mag;
    if (exp == 255) mag = 0x7c00u | ((man != 0) ? 0x200u : 0u);
    else if (e >= 31) mag = 0x7c00u;
    else if (e >= 1) mag = round_kept(((uint32_t)e << 10) | (man >> 13), 13, man);
    else if (e >= -10) mag = round_kept((man | 0x800000u) >> (126 - exp), (uint32_t)(126 - exp), man | 0x800000u);
    else mag = 0;
    return (uint16_t)(sign | mag);
}

TBO_API float tbo_f16_value(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, bits;
    float f;
    if (exp == 0) {
        float s = sign ? -1.0f : 1.0f;
        return s * (float)man * 5.9604644775390625e-8f; /* 2^-24 */
    }
    bits = (exp == 31) ? (sign | 0x7f800000u | (man << 13)) : (sign | ((exp + 112u) << 23) | (man << 13));
    memcpy(&f, &bits, 4);
    return f;
}

/* ------------------------------------------------------------------------------------------------ */
/* Reference weight / activation layouts.  crates/tachyon/src/quant.rs:47-130                        */
/* ------------------------------------------------------------------------------------------------ */

static float inverse(float d) { return d > 0.0f ? 1.0f / d : 0.0f; }

static float rte(float v) { return nearbyintf(v); } /* default rounding mode: ties to even */

/* quant.rs:71-82: the f16 scale among amax/(6 + i/4), i = 0..12, with the least squared error. */
static uint16_t q4_scale(const float *g) {
    float amax = 0.0f, best = INFINITY;
    uint16_t pick = 0;
    for (int j = 0; j < 64; j++) amax = fmaxf(amax, fabsf(g[j]));
    for (int i = 0; i < 13; i++) {
        uint16_t s = tbo_f16_bits(amax / (6.0f + (float)i / 4.0f));
        float d = tbo_f16_value(s), inv = inverse(d), err = 0.0f;
        for (int j = 0; j < 64; j++) {
            float q = fminf(fmaxf(rte(g[j] * inv), -8.0f), 7.0f);
            float e = q * d - g[j];
            err += e * e;
        }
        if (err < best) { best = err; pick = s; }
    }
    return pick;
}

/* quant.rs:47-68: Q4 packing.  w: rows*cols floats; packed: rows*cols/2 bytes; scales: rows*cols/64. */
TBO_API void tbo_q4(const float *w, size_t n, uint8_t *packed, uint16_t *scales) {
    memset(packed, 0, n / 2);
    for (size_t g = 0; g < n / 64; g++) {
        const float *grp = w + g * 64;
        scales[g] = q4_scale(grp);
        float inv = inverse(tbo_f16_value(scales[g]));
        for (int j = 0; j < 64; j++) {
            int q = (int)rte(grp[j] * inv);
            q = (q < -8 ? -8 : (q > 7 ? 7 : q)) + 8;
            packed[g * 32 + (size_t)(j / 8 * 4 + j % 4)] |= (uint8_t)(q << (j % 8 / 4 * 4));
        }
    }
}

/* quant.rs:118-130: i8 values and [s, s*sum(q)] per block of `block` values. */
TBO_API void tbo_q8_blocks(const float *x, size_t n, int block, int8_t *q, float *pairs) {
    for (size_t b = 0; b < n / (size_t)block; b++) {
        const float *v = x + b * (size_t)block;
        float amax = 0.0f;
        int32_t sum = 0;
        for (int j = 0; j < block; j++) amax = fmaxf(amax, fabsf(v[j]));
        float scale = amax / 127.0f, inv = amax > 0.0f ? 127.0f / amax : 0.0f;
        for (int j = 0; j < block; j++) {
            int8_t c = (int8_t)rte(v[j] * inv);
            q[b * (size_t)block + (size_t)j] = c;
            sum += c;
        }
        pairs[2 * b] = scale;
        pairs[2 * b + 1] = (float)sum * scale;
    }
}

/* quant.rs:102-105: the prefill pair [s, fma(s, -MAGIC, -8*s*sum)] from a [s, s*sum] pair. */
TBO_API void tbo_q8p_pairs(float *pairs, size_t blocks) {
    for (size_t b = 0; b < blocks; b++) pairs[2 * b + 1] = fmaf(pairs[2 * b], -12582912.0f, pairs[2 * b + 1] * -8.0f);
}

/* tests/common/mod.rs:95-112: the Q4 x Q8 product in f64, and the bound on its rounding error. */
TBO_API void tbo_product_q4(const uint8_t *packed, const uint16_t *scales, const float *x, size_t rows, size_t cols,
                            double *sum_out, double *bound_out) {
    int8_t *q = (int8_t *)malloc(cols);
    float *s = (float *)malloc(cols / 32 * 2 * sizeof(float));
    tbo_q8_blocks(x, cols, 32, q, s);
    for (size_t r = 0; r < rows; r++) {
        double sum = 0.0, bound = 0.0;
        for (size_t c = 0; c < cols / 32; c++) {
            double dot = 0.0;
            for (size_t j = 0; j < 32; j++) {
                size_t col = c * 32 + j, g = (r * cols + col) / 64, k = col % 64;
                int nib = (packed[g * 32 + k / 8 * 4 + k % 4] >> (k % 8 / 4 * 4)) & 15;
                dot += (double)nib * (double)q[col];
            }
            double d = (double)tbo_f16_value(scales[(r * cols + c * 32) / 64]);
            double term = d * ((double)s[2 * c] * dot - 8.0 * (double)s[2 * c + 1]);
            sum += term;
            bound += fabs(term) + d * (double)s[2 * c] * fabs(dot);
        }
        sum_out[r] = sum;
        bound_out[r] = bound;
    }
    free(q);
    free(s);
}

/* crates/tachyon/src/ptx/gemv.rs:88-110, 156-195: gemv_q4 as the GPU computes it, operation by operation.  One warp per
 * row; lane l takes the chunks of 32 weights l, l + 32, ... in rising order; a chunk adds
 * fma(fma(ss, -8, f32(sum n*q) * sx), f32(scale), sum) to the lane's f32 sum (mul.f32, fma.rn.f32, fma.rn.f32); the 32
 * sums then meet in a butterfly (shfl.bfly 16, 8, 4, 2, 1; add.f32) and lane 0 stores.  All of it is IEEE
 * round-to-nearest, so this C gives the kernel's bits. */
static void gemv_q4_lanes(const uint8_t *packed, const uint16_t *scales, const int8_t *q, const float *pairs, size_t rows, size_t cols, size_t lanes,
                          float *y) {
    size_t nch = cols / 32;
    for (size_t r = 0; r < rows; r++) {
        float lane[32];
        for (size_t l = 0; l < lanes; l++) {
            float sum = 0.0f;
            for (size_t c = l; c < nch; c += lanes) {
                int32_t acc = 0;
                for (size_t j = 0; j < 32; j++) {
                    size_t col = c * 32 + j, g = (r * cols + col) / 64, k = col % 64;
                    int nib = (packed[g * 32 + k / 8 * 4 + k % 4] >> (k % 8 / 4 * 4)) & 15;
                    acc += nib * (int32_t)q[col];
                }
                float f = (float)acc * pairs[2 * c];
                f = fmaf(pairs[2 * c + 1], -8.0f, f);
                sum = fmaf(f, tbo_f16_value(scales[(r * cols + c * 32) / 64]), sum);
            }
            lane[l] = sum;
        }
        for (size_t k = lanes / 2; k > 0; k /= 2) {
            float next[32];
            for (size_t l = 0; l < lanes; l++) next[l] = lane[l] + lane[l ^ k];
            memcpy(lane, next, sizeof lane);
        }
        y[r] = lane[0];
    }
}

TBO_API void tbo_gemv_q4(const uint8_t *packed, const uint16_t *scales, const int8_t *q, const float *pairs, size_t rows,
                         size_t cols, float *y) {
    gemv_q4_lanes(packed, scales, q, pairs, rows, cols, 32, y);
}

/* gemv_q4_narrow (ptx/gemv.rs:7-9, 156-195 with 8 lanes): rows of at most 256 weights, eight lanes a row (lane l takes chunk
 * l), the eight sums meeting in a butterfly over 4, 2 and 1.  The same steps as gemv_q4 in another order of additions. */
TBO_API void tbo_gemv_q4_narrow(const uint8_t *packed, const uint16_t *scales, const int8_t *q, const float *pairs, size_t rows,
                                size_t cols, float *y) {
    gemv_q4_lanes(packed, scales, q, pairs, rows, cols, 8, y);
}

/* Q4 weights (quant.rs:47-82) times an f32 vector that is NOT rounded to Q8 first: y[r] = sum_g d_g sum_k (n_k - 8) x_k,
 * in f64, with the sum of the terms' magnitudes as the error scale.  This is the product this build's decode path
 * computes when it is given the reference's converted weights. */
TBO_API void tbo_gemv_q4x(const uint8_t *packed, const uint16_t *scales, const float *x, size_t rows, size_t cols, double *y,
                          double *bound) {
    for (size_t r = 0; r < rows; r++) {
        double sum = 0.0, mag = 0.0;
        for (size_t g = r * cols / 64; g < (r + 1) * cols / 64; g++) {
            double d = (double)tbo_f16_value(scales[g]), t = 0.0, a = 0.0;
            for (size_t k = 0; k < 64; k++) {
                int nib = (packed[g * 32 + k / 8 * 4 + k % 4] >> (k % 8 / 4 * 4)) & 15;
                double term = (double)(nib - 8) * (double)x[g * 64 - r * cols + k];
                t += term;
                a += fabs(term);
            }
            sum += d * t;
            mag += fabs(d) * a;
        }
        y[r] = sum;
        bound[r] = mag;
    }
}

/* ------------------------------------------------------------------------------------------------ */
/* The benchmark's own weight format: int8 codes, one f16 scale per 32 along K; activation in f16 or  */
/* f32; f32 accumulation.  Follows the shape of crates/tachyon/tests/common/mod.rs:95-112 (block sums */
/* scaled per block, summed per row) with the dequantisation the benchmark configuration states.      */
/* ------------------------------------------------------------------------------------------------ */

/* y[r] = sum_b scale[r,b] * sum_{k in b} w[r,k] * x[k], accumulated in f32; also the same in f64 with the sum of
 * the terms' magnitudes (the tests' error bound).  x is f32 (an f16 input is widened by the caller, exactly). */
typedef struct { const int8_t *w; const uint16_t *scales; const float *x; size_t cols; float *y; double *exact, *bound; } gemv_job;
static void gemv_rows(void *p, long lo, long hi) {
    gemv_job *g = (gemv_job *)p;
    const int8_t *w = g->w; const uint16_t *scales = g->scales; const float *x = g->x; float *y = g->y;
    double *exact = g->exact, *bound = g->bound;
    size_t cols = g->cols, nb = cols / 32;
    for (long r = lo; r < hi; r++) {
        const int8_t *wr = w + (size_t)r * cols;
        float acc = 0.0f;
        double e = 0.0, bd = 0.0;
        for (size_t b = 0; b < nb; b++) {
            float dot = 0.0f;
            double dd = 0.0;
            for (size_t j = 0; j < 32; j++) {
                dot += (float)wr[b * 32 + j] * x[b * 32 + j];
                dd += (double)wr[b * 32 + j] * (double)x[b * 32 + j];
            }
            float s = tbo_f16_value(scales[(size_t)r * nb + b]);
            acc += s * dot;
            e += (double)s * dd;
            bd += fabs((double)s * dd);
        }
        y[r] = acc;
        if (exact) exact[r] = e;
        if (bound) bound[r] = bd;
    }
}
TBO_API void tbo_gemv_q8(const int8_t *w, const uint16_t *scales, const float *x, size_t rows, size_t cols, float *y,
                         double *exact, double *bound) {
    gemv_job g = {w, scales, x, cols, y, exact, bound};
    parallel_for((long)rows, (long)(1 + 65536 / (cols ? cols : 1)), gemv_rows, &g);
}

/* ------------------------------------------------------------------------------------------------ */
/* Small operators, in f64 as the reference's tests compute them.                                    */
/* ------------------------------------------------------------------------------------------------ */

/* tests/common/mod.rs:115-118 */
static double rms_f64(const double *x, size_t n, double eps) {
    double s = 0.0;
    for (size_t i = 0; i < n; i++) s += x[i] * x[i];
    return 1.0 / sqrt(s / (double)n + eps);
}

/* tests/common/mod.rs:121-124 (eps 1e-6 there; a parameter here) */
TBO_API void tbo_normalize(double *x, size_t n, const float *w, double eps) {
    double r = rms_f64(x, n, eps);
    for (size_t i = 0; i < n; i++) x[i] *= r * (w ? (double)w[i] : 1.0);
}

/* tests/common/mod.rs:127-134: pairs (i, i + d/2) turn by pos*freq[i], the angle formed in f32. */
TBO_API void tbo_rotate(double *x, size_t d, const float *freq, uint32_t pos) {
    size_t half = d / 2;
    for (size_t i = 0; i < half; i++) {
        float ang = (float)pos * freq[i];
        double s = sin((double)ang), c = cos((double)ang), a = x[i], b = x[i + half];
        x[i] = a * c - b * s;
        x[i + half] = b * c + a * s;
    }
}

/* ptx/attend.rs:62-65: freq[i] = theta^(-2i/d) for i < fraction*d/2, else 0. */
TBO_API void tbo_rope_freq(float theta, int d, float fraction, float *freq) {
    int turned = (int)(fraction * (float)(d / 2));
    for (int i = 0; i < d / 2; i++) freq[i] = i < turned ? powf(theta, -((float)(2 * i)) / (float)d) : 0.0f;
}

/* tests/decode.rs:26-28 */
TBO_API double tbo_gelu_tanh(double x) { return 0.5 * x * (1.0 + tanh(sqrt(2.0 / M_PI) * (x + 0.044715 * x * x * x))); }

/* tests/decode.rs:84-97: h' = (h + w1*rmsnorm(y))*scale when y is given; x = w2*rmsnorm(h') (or h' when w2 is
 * absent).  One chunk of `n` values. */
TBO_API void tbo_norm_step(const float *h, const float *y, const float *w1, const float *w2, size_t n, double eps,
                           double scale, double *h_out, double *x_out) {
    for (size_t i = 0; i < n; i++) h_out[i] = (double)h[i];
    if (y) {
        double s = 0.0;
        for (size_t i = 0; i < n; i++) s += (double)y[i] * (double)y[i];
        double r = 1.0 / sqrt(s / (double)n + eps);
        for (size_t i = 0; i < n; i++) h_out[i] = (h_out[i] + (double)y[i] * r * (double)w1[i]) * scale;
    }
    double r = w2 ? rms_f64(h_out, n, eps) : 1.0;
    for (size_t i = 0; i < n; i++) x_out[i] = h_out[i] * r * (w2 ? (double)w2[i] : 1.0);
}

/* tests/common/mod.rs:137-143: softmax(scale * q.k) . v over n positions; keys/values given as rows of d. */
static void attention_f64(const double *q, const double *k, const double *v, size_t n, size_t d, double scale, double *out) {
    double *p = (double *)malloc(n * sizeof(double)), m = -INFINITY, z = 0.0;
    for (size_t t = 0; t < n; t++) {
        double s = 0.0;
        for (size_t i = 0; i < d; i++) s += q[i] * k[t * d + i];
        p[t] = s * scale;
        if (p[t] > m) m = p[t];
    }
    for (size_t t = 0; t < n; t++) { p[t] = exp(p[t] - m); z += p[t]; }
    for (size_t i = 0; i < d; i++) {
        double o = 0.0;
        for (size_t t = 0; t < n; t++) o += p[t] * v[t * d + i];
        out[i] = o / z;
    }
    free(p);
}

/*
 * Decode attention for one new token.  tests/decode.rs:258-285 (ring indexing (cur + cap - age) % cap, the
 * fresh token's key/value taken from the projections, not the cache) with ptx/attend.rs:1-32's options.
 *   qkv    f32 [(heads + 2*kv_heads) * d]: query heads, then (when fresh) key heads, then value heads
 *   qn, kn per-head norm weights [d], or NULL for "no norms" (plain mode: q, k, v used as given, no RoPE when
 *          freq is NULL)
 *   kc, vc f16 caches [kv_heads][cap][d]; when `fresh`, the new key/value are written at slot pos % cap
 *   out    f64 [heads * d]
 * Attends the newest min(pos + 1, window) positions with softmax scale `scale`.
 */
TBO_API void tbo_attend_decode(const float *qkv, const float *qn, const float *kn, const float *freq, uint16_t *kc,
                               uint16_t *vc, uint32_t pos, uint32_t cap, uint32_t window, int fresh, int heads,
                               int kv_heads, int d, double scale, double eps, double *out) {
    size_t n = (pos + 1 < window) ? pos + 1 : window, cur = pos % cap;
    int group = heads / kv_heads;
    double *keys = (double *)malloc(n * (size_t)d * sizeof(double)), *vals = (double *)malloc(n * (size_t)d * sizeof(double));
    double *q = (double *)malloc((size_t)d * sizeof(double));
    for (int g = 0; g < kv_heads; g++) {
        double *k = NULL, *v = NULL;
        if (fresh) {
            k = (double *)malloc((size_t)d * sizeof(double));
            v = (double *)malloc((size_t)d * sizeof(double));
            for (int i = 0; i < d; i++) {
                k[i] = (double)qkv[(size_t)(heads + g) * (size_t)d + (size_t)i];
                v[i] = (double)qkv[(size_t)(heads + kv_heads + g) * (size_t)d + (size_t)i];
            }
            if (kn) tbo_normalize(k, (size_t)d, kn, eps);
            if (freq) tbo_rotate(k, (size_t)d, freq, pos);
            if (kn) tbo_normalize(v, (size_t)d, NULL, eps);
        }
        for (size_t age = 0; age < n; age++) {
            size_t t = (cur + cap - age) % cap;
            for (int i = 0; i < d; i++) {
                size_t at = ((size_t)g * cap + t) * (size_t)d + (size_t)i;
                keys[age * (size_t)d + (size_t)i] = (fresh && t == cur) ? k[i] : (double)tbo_f16_value(kc[at]);
                vals[age * (size_t)d + (size_t)i] = (fresh && t == cur) ? v[i] : (double)tbo_f16_value(vc[at]);
            }
        }
        for (int h = group * g; h < group * (g + 1); h++) {
            for (int i = 0; i < d; i++) q[i] = (double)qkv[(size_t)h * (size_t)d + (size_t)i];
            if (qn) tbo_normalize(q, (size_t)d, qn, eps);
            if (freq) tbo_rotate(q, (size_t)d, freq, pos);
            attention_f64(q, keys, vals, n, (size_t)d, scale, out + (size_t)h * (size_t)d);
        }
        if (fresh) {
            for (int i = 0; i < d; i++) {
                size_t at = ((size_t)g * cap + cur) * (size_t)d + (size_t)i;
                kc[at] = tbo_f16_bits((float)k[i]);
                vc[at] = tbo_f16_bits((float)v[i]);
            }
            free(k);
            free(v);
        }
    }
    free(keys);
    free(vals);
    free(q);
}

/* ------------------------------------------------------------------------------------------------ */
/* Sampler, greedy part.  tests/sample.rs:61-73 (transform) and :100 (largest value, lowest index).   */
/* ------------------------------------------------------------------------------------------------ */

TBO_API double tbo_sample_transform(float x, size_t i, float softcap, float penalty, float temperature, const uint32_t *seen,
                                    const uint32_t *allowed) {
    double v = (double)x;
    if (softcap > 0.0f) v = (double)softcap * tanh(v / (double)softcap);
    if (allowed && !((allowed[i / 32] >> (i % 32)) & 1u)) return -INFINITY;
    if (seen && ((seen[i / 32] >> (i % 32)) & 1u)) v = v > 0.0 ? v / (double)penalty : v * (double)penalty;
    return temperature > 0.0f ? v / (double)temperature : v;
}

/* Returns the greedy pick; when `gap` is given it receives best minus runner-up (the "top-2 gap"). */
TBO_API uint32_t tbo_sample_greedy(const float *logits, size_t vocab, float softcap, float penalty, const uint32_t *seen,
                                   const uint32_t *allowed, double *gap) {
    size_t best = 0;
    double bv = -INFINITY, second = -INFINITY;
    for (size_t i = 0; i < vocab; i++) {
        double v = tbo_sample_transform(logits[i], i, softcap, penalty, 0.0f, seen, allowed);
        if (i == 0 || v > bv) { second = bv; bv = v; best = i; }
        else if (v > second) second = v;
    }
    if (gap) *gap = bv - second;
    return (uint32_t)best;
}

/* The k largest transformed logits, largest first, lower index first among equals. */
TBO_API void tbo_sample_topk(const float *logits, size_t vocab, int k, uint32_t *idx, float *val) {
    for (int j = 0; j < k; j++) { idx[j] = 0xffffffffu; val[j] = -INFINITY; }
    for (size_t i = 0; i < vocab; i++) {
        float v = logits[i];
        int at = k;
        while (at > 0 && (v > val[at - 1] || (v == val[at - 1] && (uint32_t)i < idx[at - 1]))) at--;
        if (at < k) {
            for (int j = k - 1; j > at; j--) { val[j] = val[j - 1]; idx[j] = idx[j - 1]; }
            val[at] = v;
            idx[at] = (uint32_t)i;
        }
    }
}

/* ------------------------------------------------------------------------------------------------ */
/* Sampler, drawing part: ptx/sample.rs:81-88 (hash), 113-121 (Gumbel noise), 318-352 (filter check    */
/* and redraw), with the transcendental steps in double instead of the GPU's approximate instructions. */
/* ------------------------------------------------------------------------------------------------ */

typedef struct {   /* ptx/sample.rs:38-78, the 40 bytes the kernel reads */
    float softcap, temperature, top_p, min_p, penalty;
    uint32_t top_k;
    uint64_t allowed, seed;
} tbo_sampling;

static uint32_t fmix32(uint32_t h) { h ^= h >> 16; h *= 0x85EBCA6Bu; h ^= h >> 13; h *= 0xC2B2AE35u; h ^= h >> 16; return h; }
static uint32_t noise_base(uint32_t step, uint32_t round, uint64_t seed) {
    uint32_t h = step * 0x9E3779B9u + (uint32_t)(seed >> 32);
    h = round * 0x85EBCA77u + h;
    return fmix32(fmix32(h) ^ (uint32_t)seed);
}
static double gumbel_noise(uint32_t i, uint32_t base) {
    uint32_t h = fmix32((i * 0x9E3779B9u) ^ base) >> 9;
    double u = ((double)h + 0.5) * 0x1p-23;
    return -log(-log(u));
}

/* One draw at step `step` (the kernel's state[0]); `allowed`, `seen`: bitmaps or NULL.  `rounds` receives the number of
 * failed draws. */
TBO_API uint32_t tbo_sample_draw(const float *logits, size_t vocab, const tbo_sampling *c, uint32_t step, const uint32_t *seen,
                                 const uint32_t *allowed, int *rounds) {
    double *x = (double *)malloc(vocab * sizeof(double));
    double m = -INFINITY, z = 0.0;
    size_t amax = 0;
    for (size_t i = 0; i < vocab; i++) {
        x[i] = tbo_sample_transform(logits[i], i, c->softcap, c->penalty, c->temperature, seen, allowed);
        if (i == 0 || x[i] > m) { m = x[i]; amax = i; }
    }
    uint32_t token = (uint32_t)amax;
    int round = 0;
    if (c->temperature > 0.0f) {
        for (size_t i = 0; i < vocab; i++) z += exp(x[i] - m);
        int filter = c->top_k != 0 || c->top_p < 1.0f || c->min_p > 0.0f;
        double thr = -INFINITY;
        for (;;) {
            uint32_t base = noise_base(step, (uint32_t)round, c->seed);
            double kv = -INFINITY;
            size_t ki = amax;
            for (size_t i = 0; i < vocab; i++) {
                if (!(x[i] > thr)) continue;
                double k = x[i] + gumbel_noise((uint32_t)i, base);
                if (k > kv) { kv = k; ki = i; }
            }
            token = (uint32_t)ki;
            if (!filter) break;
            double cnt = 0.0, mass = 0.0, lj = x[ki];
            for (size_t i = 0; i < vocab; i++) if (x[i] > lj) { cnt += 1.0; mass += exp(x[i] - m); }
            int ok = (c->top_k == 0 || cnt < (double)c->top_k) && (c->top_p >= 1.0f || mass < (double)c->top_p * z || mass == 0.0) &&
                     lj - m >= log((double)c->min_p);
            if (ok) break;
            thr = lj;
            round++;
            token = (uint32_t)amax;
            if (round >= 32) break;
        }
    }
    if (rounds) *rounds = round;
    free(x);
    return token;
}

/* ------------------------------------------------------------------------------------------------ */
/* Seeded synthetic tensors.  The reference's benches use synthetic weights too (benches/gemv.rs:8-9); */
/* these generators are this build's own and use only exactly-rounded operations, so a GPU fill kernel */
/* written with the same steps produces identical bits.                                               */
/* ------------------------------------------------------------------------------------------------ */

static inline uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

static inline uint64_t draw(uint64_t seed, uint64_t stream, uint64_t i) {
    return mix64(mix64(seed + 0x9E3779B97F4A7C15ull * (stream + 1)) + i);
}

/* Approximately N(0,1): twelve 16-bit uniforms from three draws, summed exactly. */
static inline float gauss(uint64_t seed, uint64_t stream, uint64_t i) {
    uint32_t sum = 0;
    for (int j = 0; j < 3; j++) {
        uint64_t h = draw(seed, stream, 3 * i + (uint64_t)j);
        sum += (uint32_t)(h & 0xffff) + (uint32_t)((h >> 16) & 0xffff) + (uint32_t)((h >> 32) & 0xffff) + (uint32_t)(h >> 48);
    }
    return ((float)sum - 393210.0f) * (1.0f / 65536.0f);
}

/* int8 codes uniform in [-127, 127]. */
typedef struct { uint64_t seed, stream; void *out; float mul; int kind; } fill_job;
static void fill_range(void *p, long lo, long hi) {
    fill_job *f = (fill_job *)p;
    for (long i = lo; i < hi; i++) {
        if (f->kind == 0) ((int8_t *)f->out)[i] = (int8_t)((int)(draw(f->seed, f->stream, (uint64_t)i) % 255u) - 127);
        else if (f->kind == 1) ((uint16_t *)f->out)[i] = tbo_f16_bits(fabsf(gauss(f->seed, f->stream, (uint64_t)i)) * f->mul);
        else ((uint16_t *)f->out)[i] = tbo_f16_bits(gauss(f->seed, f->stream, (uint64_t)i) * f->mul);
    }
}
TBO_API void tbo_fill_codes(uint64_t seed, uint64_t stream, int8_t *w, size_t n) {
    fill_job f = {seed, stream, w, 0.0f, 0};
    parallel_for((long)n, 1 << 16, fill_range, &f);
}

/* f16 scales |N(0,1)| * mul. */
TBO_API void tbo_fill_scales(uint64_t seed, uint64_t stream, uint16_t *s, size_t n, float mul) {
    fill_job f = {seed, stream, s, mul, 1};
    parallel_for((long)n, 1 << 14, fill_range, &f);
}

/* f32 values lo + (hi - lo) * u, u uniform in [0, 1) with 16 bits. */
TBO_API void tbo_fill_uniform(uint64_t seed, uint64_t stream, float *x, size_t n, float lo, float hi) {
    for (size_t i = 0; i < n; i++) x[i] = fmaf((float)(draw(seed, stream, (uint64_t)i) & 0xffff), (hi - lo) * (1.0f / 65536.0f), lo);
}

/* f16 values N(0,1) * mul. */
TBO_API void tbo_fill_gauss_f16(uint64_t seed, uint64_t stream, uint16_t *x, size_t n, float mul) {
    fill_job f = {seed, stream, x, mul, 2};
    parallel_for((long)n, 1 << 14, fill_range, &f);
}

/* f32 values N(0,1) * mul. */
TBO_API void tbo_fill_gauss_f32(uint64_t seed, uint64_t stream, float *x, size_t n, float mul) {
    for (size_t i = 0; i < n; i++) x[i] = gauss(seed, stream, (uint64_t)i) * mul;
}

/* ------------------------------------------------------------------------------------------------ */
/* The decoder forward pass, f32, one token at a time.  crates/tachyon/tests/common/tiny.rs:225-386   */
/* for a model without per-layer inputs, shared caches or experts (its DENSE path, :233-238, 263-299). */
/* Weights are this build's Q8 layout (int8 codes + f16 scale per 32), dequantised on the fly.         */
/* ------------------------------------------------------------------------------------------------ */

typedef struct {
    int32_t hidden, ffn, heads, kv_heads, head_dim, vocab, layers, window, context;
    float theta_sliding, theta_global, fraction_global, eps, softcap, attn_scale, embed_scale;
    int32_t weight_bits; /* 0 or 8: int8 codes, a scale per 32; 4: the reference's Q4 (quant.rs:47-82), a scale per 64 */
    int32_t global_head_dim, global_kv_heads; /* Config::head_dim[1], Config::kv_heads[1] (model/mod.rs:34-37); 0 = as the sliding layers */
    int32_t per_layer;                        /* Config::per_layer: width of each layer's per-layer input; 0 = none */
} tbo_config;

typedef struct {
    const int8_t *qkv, *o, *gate_up, *down;          /* codes: [(h+2kv)*d, hidden], [hidden, h*d], [2*ffn, hidden] (gate rows, then up), [hidden, ffn] */
    const uint16_t *qkv_s, *o_s, *gate_up_s, *down_s; /* f16 scales, one per 32 along the row */
    const float *q_norm, *k_norm, *input_ln, *post_attn_ln, *pre_ffn_ln, *post_ffn_ln;
    float layer_scalar;
    int32_t global;
    uint16_t *kc, *vc;                                /* f16 caches [kv_heads][cap][head_dim]; cap = context (global) or ring */
    int32_t cap;
    int32_t shared;                                   /* != 0: no key/value rows in qkv; kc, vc are another layer's (tiny.rs: Config::source) */
    const int8_t *pl_gate, *pl_proj;                  /* per-layer input: gate [per_layer, hidden], projection [hidden, per_layer] */
    const uint16_t *pl_gate_s, *pl_proj_s;
    const float *post_pl_ln;                          /* post_per_layer_input_norm [hidden] */
} tbo_layer;

typedef struct {
    tbo_config cfg;
    const int8_t *embed;      /* [vocab, hidden] */
    const uint16_t *embed_s;
    const float *norm;        /* [hidden] */
    tbo_layer *layers;
    const int8_t *embed_pl, *pl_model_proj; /* per-layer table [vocab, layers*per_layer]; projection of the embedding [layers*per_layer, hidden] */
    const uint16_t *embed_pl_s, *pl_model_proj_s;
    const float *pl_norm;                   /* per_layer_projection_norm [per_layer] */
} tbo_model;

static int nibble(const uint8_t *packed, size_t at) { /* weight `at` of a row-major Q4 matrix, 0..15 (quant.rs:60-66) */
    size_t g = at / 64, k = at % 64;
    return (packed[g * 32 + k / 8 * 4 + k % 4] >> (k % 8 / 4 * 4)) & 15;
}

/* y = W x for the model's weight format, accumulated in f32 group by group. */
static void matvec(const tbo_config *c, const int8_t *w, const uint16_t *s, const float *x, size_t rows, size_t cols, float *y) {
    if (c->weight_bits != 4) {
        tbo_gemv_q8(w, s, x, rows, cols, y, NULL, NULL);
        return;
    }
    const uint8_t *packed = (const uint8_t *)w;
    for (size_t r = 0; r < rows; r++) {
        float sum = 0.0f;
        for (size_t g = 0; g < cols / 64; g++) {
            float t = 0.0f;
            for (size_t k = 0; k < 64; k++) t += (float)(nibble(packed, r * cols + g * 64 + k) - 8) * x[g * 64 + k];
            sum += tbo_f16_value(s[r * cols / 64 + g]) * t;
        }
        y[r] = sum;
    }
}

/* tiny.rs:364-367: x / sqrt(mean(x^2) + eps), times w when given, in f32. */
static void rms_f32(const float *x, const float *w, size_t n, float eps, float *out) {
    float s = 0.0f;
    for (size_t i = 0; i < n; i++) s += x[i] * x[i];
    float r = 1.0f / sqrtf(s / (float)n + eps);
    for (size_t i = 0; i < n; i++) out[i] = x[i] * r * (w ? w[i] : 1.0f);
}

/* tiny.rs:370-380: rotate_half RoPE in f32. */
static void rotate_f32(float *x, size_t d, const float *freq, uint32_t pos) {
    size_t half = d / 2;
    for (size_t j = 0; j < half; j++) {
        float ang = (float)pos * freq[j], s = sinf(ang), c = cosf(ang), a = x[j], b = x[j + half];
        x[j] = a * c - b * s;
        x[j + half] = b * c + a * s;
    }
}

/* tiny.rs:382-384 */
static float gelu_f32(float x) { return 0.5f * x * (1.0f + tanhf(sqrtf(2.0f / (float)M_PI) * (x + 0.044715f * x * x * x))); }

/* One token through the model at `pos`; logits (before soft-capping) into `logits` [vocab] when not NULL.
 * Returns the greedy token (soft cap applied first, as the sampler does).  `stop_layer` > 0 stops after that many
 * layers and skips the head (for timing a bounded sample); hidden state is left in `h_out` when given. */
TBO_API int32_t tbo_decoder_step(tbo_model *m, uint32_t token, uint32_t pos, float *logits, int stop_layer, float *h_out) {
    const tbo_config *c = &m->cfg;
    size_t H = (size_t)c->hidden, F = (size_t)c->ffn;
    size_t Dg = (size_t)(c->global_head_dim ? c->global_head_dim : c->head_dim), KVg = (size_t)(c->global_kv_heads ? c->global_kv_heads : c->kv_heads);
    size_t Dmax = Dg > (size_t)c->head_dim ? Dg : (size_t)c->head_dim;
    size_t nq_max = (size_t)c->heads * Dmax, nkv_max = (KVg * Dg > (size_t)c->kv_heads * (size_t)c->head_dim) ? KVg * Dg : (size_t)c->kv_heads * (size_t)c->head_dim;
    float *x = (float *)malloc(H * 4), *h = (float *)malloc(H * 4), *qkv = (float *)malloc((nq_max + 2 * nkv_max) * 4);
    float *att = (float *)malloc(nq_max * 4), *y = (float *)malloc(H * 4), *gu = (float *)malloc(2 * F * 4), *a = (float *)malloc(F * 4);
    float *freq = (float *)malloc(Dmax / 2 * 4), *tmp = (float *)malloc(Dmax * 4);
    /* tiny.rs:233: the embedding row times sqrt(hidden) (model/decode.rs:571 rounds that factor to bfloat16; the caller
     * passes the factor it wants in embed_scale). */
    for (size_t i = 0; i < H; i++) {
        size_t at = (size_t)token * H + i;
        if (c->weight_bits == 4) x[i] = (float)(nibble((const uint8_t *)m->embed, at) - 8) * tbo_f16_value(m->embed_s[at / 64]) * c->embed_scale;
        else x[i] = (float)m->embed[at] * tbo_f16_value(m->embed_s[at / 32]) * c->embed_scale;
    }
    /* tiny.rs:239-252: every layer's input (rmsnorm(projection of the embedding / sqrt(hidden)) + table row * sqrt(per_layer)) / sqrt(2). */
    size_t PL = (size_t)c->per_layer, PLW = PL * (size_t)c->layers;
    float *pli = NULL;
    if (PL) {
        float *proj = (float *)malloc(PLW * 4);
        pli = (float *)malloc(PLW * 4);
        matvec(c, m->pl_model_proj, m->pl_model_proj_s, x, PLW, H, proj);
        for (size_t i = 0; i < PLW; i++) proj[i] /= sqrtf((float)H);
        for (size_t l = 0; l < (size_t)c->layers; l++) {
            rms_f32(proj + l * PL, m->pl_norm, PL, c->eps, pli + l * PL);
            for (size_t i = 0; i < PL; i++) {
                size_t at = (size_t)token * PLW + l * PL + i;
                float e = c->weight_bits == 4 ? (float)(nibble((const uint8_t *)m->embed_pl, at) - 8) * tbo_f16_value(m->embed_pl_s[at / 64]) * sqrtf((float)PL)
                                              : (float)m->embed_pl[at] * tbo_f16_value(m->embed_pl_s[at / 32]) * sqrtf((float)PL);
                pli[l * PL + i] = (pli[l * PL + i] + e) * 0.70710678118654752f;
            }
        }
        free(proj);
    }
    int nl = stop_layer > 0 ? stop_layer : c->layers;
    for (int li = 0; li < nl; li++) {
        tbo_layer *L = &m->layers[li];
        size_t D = L->global ? Dg : (size_t)c->head_dim, kvh = L->global ? KVg : (size_t)c->kv_heads; /* this kind's head size and key-value heads */
        size_t nq = (size_t)c->heads * D, nkv = kvh * D;
        tbo_rope_freq(L->global ? c->theta_global : c->theta_sliding, (int)D, L->global ? c->fraction_global : 1.0f, freq);
        rms_f32(x, L->input_ln, H, c->eps, h);                                  /* tiny.rs:278 */
        matvec(c, L->qkv, L->qkv_s, h, nq + (L->shared ? 0 : 2 * nkv), H, qkv);  /* :279, 286-287 (fused q, k, v) */
        for (int hd = 0; hd < c->heads; hd++) {                                 /* :280-283 */
            rms_f32(qkv + (size_t)hd * D, L->q_norm, D, c->eps, tmp);
            rotate_f32(tmp, D, freq, pos);
            memcpy(qkv + (size_t)hd * D, tmp, D * 4);
        }
        uint32_t cap = (uint32_t)L->cap, slot = pos % cap;
        for (int g = 0; g < (L->shared ? 0 : (int)kvh); g++) {                  /* :288-289: k-norm + RoPE, v-norm without weights */
            rms_f32(qkv + nq + (size_t)g * D, L->k_norm, D, c->eps, tmp);
            rotate_f32(tmp, D, freq, pos);
            for (size_t i = 0; i < D; i++) L->kc[((size_t)g * cap + slot) * D + i] = tbo_f16_bits(tmp[i]);
            rms_f32(qkv + nq + nkv + (size_t)g * D, NULL, D, c->eps, tmp);
            for (size_t i = 0; i < D; i++) L->vc[((size_t)g * cap + slot) * D + i] = tbo_f16_bits(tmp[i]);
        }
        /* :291-292, 340-357: each query head attends the newest min(pos+1, window) positions of its kv head.  The cache
         * holds f16 (model/decode.rs keeps it so); the reference's f32 test model keeps f32. */
        uint32_t win = L->global ? (uint32_t)c->context : (uint32_t)c->window;
        size_t n = (pos + 1 < win) ? pos + 1 : win;
        int group = c->heads / (int)kvh;
        for (int hd = 0; hd < c->heads; hd++) {
            int g = hd / group;
            float *sc = (float *)malloc(n * 4), mx = -INFINITY, sum = 0.0f;
            const float *q = qkv + (size_t)hd * D;
            for (size_t age = 0; age < n; age++) {
                size_t t = (slot + cap - age) % cap;
                const uint16_t *kr = L->kc + ((size_t)g * cap + t) * D;
                float s = 0.0f;
                for (size_t i = 0; i < D; i++) s += q[i] * tbo_f16_value(kr[i]);
                sc[age] = s * c->attn_scale;
                mx = fmaxf(mx, sc[age]);
            }
            for (size_t age = 0; age < n; age++) { sc[age] = expf(sc[age] - mx); sum += sc[age]; }
            float *o = att + (size_t)hd * D;
            for (size_t i = 0; i < D; i++) o[i] = 0.0f;
            for (size_t age = 0; age < n; age++) {
                size_t t = (slot + cap - age) % cap;
                const uint16_t *vr = L->vc + ((size_t)g * cap + t) * D;
                float p = sc[age] / sum;
                for (size_t i = 0; i < D; i++) o[i] += p * tbo_f16_value(vr[i]);
            }
            free(sc);
        }
        matvec(c, L->o, L->o_s, att, H, nq, y);                                  /* :294 */
        rms_f32(y, L->post_attn_ln, H, c->eps, h);
        for (size_t i = 0; i < H; i++) x[i] += h[i];
        rms_f32(x, L->pre_ffn_ln, H, c->eps, h);                                 /* :312 */
        matvec(c, L->gate_up, L->gate_up_s, h, 2 * F, H, gu);
        for (size_t i = 0; i < F; i++) a[i] = gelu_f32(gu[i]) * gu[F + i];       /* :309 */
        matvec(c, L->down, L->down_s, a, H, F, y);
        rms_f32(y, L->post_ffn_ln, H, c->eps, h);                                /* :314 */
        if (PL) {                                                                /* :298-300: gelu(gate x) * input, projected back, normed, added */
            for (size_t i = 0; i < H; i++) x[i] += h[i];
            float *g = (float *)malloc(PL * 4);
            matvec(c, L->pl_gate, L->pl_gate_s, x, PL, H, g);
            for (size_t i = 0; i < PL; i++) g[i] = gelu_f32(g[i]) * pli[(size_t)li * PL + i];
            matvec(c, L->pl_proj, L->pl_proj_s, g, H, PL, y);
            free(g);
            rms_f32(y, L->post_pl_ln, H, c->eps, h);
        }
        for (size_t i = 0; i < H; i++) x[i] = (x[i] + h[i]) * L->layer_scalar;   /* :296-297, 301 */
    }
    int32_t pick = -1;
    if (h_out) memcpy(h_out, x, H * 4);
    if (stop_layer <= 0) {
        float *lg = logits ? logits : (float *)malloc((size_t)c->vocab * 4);
        rms_f32(x, m->norm, H, c->eps, h);                                       /* :238 */
        matvec(c, m->embed, m->embed_s, h, (size_t)c->vocab, H, lg);
        pick = (int32_t)tbo_sample_greedy(lg, (size_t)c->vocab, c->softcap, 1.0f, NULL, NULL, NULL);
        if (!logits) free(lg);
    }
    free(x); free(h); free(qkv); free(att); free(y); free(gu); free(a); free(freq); free(tmp); free(pli);
    return pick;
}

TBO_API int tbo_threads(void) { return threads_now(); }

TBO_API void tbo_set_threads(int n) { g_threads = n > 256 ? 256 : n; }

/* ------------------------------------------------------------------------------------------------ */
/* The ModernBERT-style encoder forward, f32, one sequence.  crates/tachyon/tests/encoder.rs:29-123    */
/* (linear, norm, erf to 1.5e-7 by Abramowitz-Stegun 7.1.26, gelu, attend with RoPE and window, encode). */
/* Pinned by the reference's tiny-encoder fixture (PyTorch hidden states), see tests/golden.           */
/* ------------------------------------------------------------------------------------------------ */

typedef struct {
    int32_t hidden, heads, inter, vocab, layers, window, gated;
    float theta_global, theta_local, eps;
    const uint8_t *global; /* [layers] */
} tbo_enc_config;

typedef struct {
    const float *attn_norm; /* NULL in layer 0 */
    const float *qkv, *o, *mlp_norm, *up, *down;
} tbo_enc_layer;

/* encoder.rs:29-35 (no bias) */
static void enc_linear(const float *x, const float *w, size_t n, size_t cols, size_t out, float *y) {
    for (size_t r = 0; r < n; r++)
        for (size_t o = 0; o < out; o++) {
            float s = 0.0f;
            for (size_t c = 0; c < cols; c++) s += x[r * cols + c] * w[o * cols + c];
            y[r * out + o] = s;
        }
}

/* encoder.rs:38-48 */
static void enc_norm(const float *x, const float *w, size_t n, size_t h, float eps, float *y) {
    for (size_t r = 0; r < n; r++) {
        float mean = 0.0f, var = 0.0f;
        for (size_t i = 0; i < h; i++) mean += x[r * h + i];
        mean /= (float)h;
        for (size_t i = 0; i < h; i++) var += (x[r * h + i] - mean) * (x[r * h + i] - mean);
        var /= (float)h;
        float rs = 1.0f / sqrtf(var + eps);
        for (size_t i = 0; i < h; i++) y[r * h + i] = (x[r * h + i] - mean) * rs * w[i];
    }
}

/* encoder.rs:51-59 */
TBO_API float tbo_erf_as(float x) {
    float t = 1.0f / (1.0f + 0.3275911f * fabsf(x));
    float p = t * (0.2548296f + t * (-0.28449674f + t * (1.4214137f + t * (-1.4531521f + t * 1.0614054f))));
    return copysignf(1.0f - p * expf(-x * x), x);
}
static float enc_gelu(float x) { return 0.5f * x * (1.0f + tbo_erf_as(x / 1.41421356237f)); }
/* tests/encoder.rs:64-66 */
static float enc_silu(float x) { return x / (1.0f + expf(-x)); }

/* encoder.rs:67-101: RoPE by row index, window |i - j| <= w or none (w < 0), scale 1/sqrt(d). */
static void enc_attend(const float *qkv, size_t n, size_t heads, size_t d, long window, float theta, float *out) {
    size_t h = heads * d;
    float *q = (float *)malloc(n * h * 4), *k = (float *)malloc(n * h * 4), *sc = (float *)malloc(n * 4);
    for (size_t r = 0; r < n; r++)
        for (int part = 0; part < 2; part++) {
            float *dst = (part ? k : q) + r * h;
            memcpy(dst, qkv + r * 3 * h + (size_t)part * h, h * 4);
            for (size_t hd = 0; hd < heads; hd++)
                for (size_t j = 0; j < d / 2; j++) {
                    float ang = (float)r * powf(theta, -2.0f * (float)j / (float)d), c = cosf(ang), s = sinf(ang);
                    float a = dst[hd * d + j], b = dst[hd * d + j + d / 2];
                    dst[hd * d + j] = a * c - b * s;
                    dst[hd * d + j + d / 2] = b * c + a * s;
                }
        }
    memset(out, 0, n * h * 4);
    for (size_t i = 0; i < n; i++)
        for (size_t hd = 0; hd < heads; hd++) {
            float top = -INFINITY, sum = 0.0f;
            for (size_t j = 0; j < n; j++) {
                long dist = (long)i - (long)j;
                if (window >= 0 && (dist > window || -dist > window)) { sc[j] = -INFINITY; continue; }
                float s = 0.0f;
                for (size_t t = 0; t < d; t++) s += q[i * h + hd * d + t] * k[j * h + hd * d + t];
                sc[j] = s / sqrtf((float)d);
                if (sc[j] > top) top = sc[j];
            }
            for (size_t j = 0; j < n; j++) { sc[j] = sc[j] == -INFINITY ? 0.0f : expf(sc[j] - top); sum += sc[j]; }
            for (size_t j = 0; j < n; j++) {
                if (sc[j] == 0.0f) continue;
                float p = sc[j] / sum;
                for (size_t t = 0; t < d; t++) out[i * h + hd * d + t] += p * qkv[j * 3 * h + 2 * h + hd * d + t];
            }
        }
    free(q); free(k); free(sc);
}

/* The 8-bit product on Q8E activations and weights (codes, an f32 scale per 64 along a row), sum by sum as the reference's
 * gemm_q8 kernel forms it (crates/tachyon/src/ptx/encoder.rs:315-375): per group of 64 the integer sum i, read as the
 * float 12582912 + i (exact: |i| < 2^22), then f = fma(12582912 + i, sa, -12582912 sa) and c = fma(f, sw, c), the groups
 * in order; the bias is added at the store (encoder.rs:418-436).  y: f32 [tokens, rows], before any activation. */
TBO_API void tbo_gemm_q8e(const int8_t *a, const float *sa, const int8_t *w, const float *sw, const float *bias, size_t tokens, size_t rows, size_t cols,
                          float *y) {
    size_t groups = cols / 64;
    for (size_t t = 0; t < tokens; t++)
        for (size_t r = 0; r < rows; r++) {
            float c = 0.0f;
            for (size_t g = 0; g < groups; g++) {
                int32_t i = 0;
                for (size_t k = 0; k < 64; k++) i += (int32_t)a[t * cols + g * 64 + k] * (int32_t)w[r * cols + g * 64 + k];
                float ts = sa[t * groups + g], tz = ts * -12582912.0f;
                float f = fmaf(12582912.0f + (float)i, ts, tz);
                c = fmaf(f, sw[r * groups + g], c);
            }
            y[t * rows + r] = c + (bias ? bias[r] : 0.0f);
        }
}

/* encoder.rs:104-123.  gated: Wi is [2*inter, h] and the MLP is gelu(first half) * second half (2: silu); otherwise Wi is
 * [inter, h] and the MLP is gelu(Wi x) (the benchmark's plain GeLU FFN).  hidden_out: [n, hidden]. */
TBO_API void tbo_encoder_forward(const tbo_enc_config *c, const float *embed, const float *embed_norm, const tbo_enc_layer *layers,
                                 const float *final_norm, const uint32_t *ids, size_t n, float *hidden_out) {
    size_t h = (size_t)c->hidden, inter = (size_t)c->inter, d = h / (size_t)c->heads, up_rows = c->gated ? 2 * inter : inter;
    float *x = (float *)malloc(n * h * 4), *a = (float *)malloc(n * h * 4), *qkv = (float *)malloc(n * 3 * h * 4);
    float *att = (float *)malloc(n * h * 4), *up = (float *)malloc(n * up_rows * 4), *g = (float *)malloc(n * inter * 4);
    for (size_t r = 0; r < n; r++) memcpy(a + r * h, embed + (size_t)ids[r] * h, h * 4);
    enc_norm(a, embed_norm, n, h, c->eps, x);
    for (int l = 0; l < c->layers; l++) {
        const tbo_enc_layer *L = &layers[l];
        if (L->attn_norm) enc_norm(x, L->attn_norm, n, h, c->eps, a);
        else memcpy(a, x, n * h * 4);
        enc_linear(a, L->qkv, n, h, 3 * h, qkv);
        int global = c->global[l] != 0;
        enc_attend(qkv, n, (size_t)c->heads, d, global ? -1 : (long)c->window, global ? c->theta_global : c->theta_local, att);
        enc_linear(att, L->o, n, h, h, a);
        for (size_t i = 0; i < n * h; i++) x[i] += a[i];
        enc_norm(x, L->mlp_norm, n, h, c->eps, a);
        enc_linear(a, L->up, n, h, up_rows, up);
        for (size_t r = 0; r < n; r++)
            for (size_t i = 0; i < inter; i++)
                g[r * inter + i] = c->gated == 2 ? enc_silu(up[r * up_rows + i]) * up[r * up_rows + inter + i]
                                 : c->gated    ? enc_gelu(up[r * up_rows + i]) * up[r * up_rows + inter + i] : enc_gelu(up[r * up_rows + i]);
        enc_linear(g, L->down, n, inter, h, a);
        for (size_t i = 0; i < n * h; i++) x[i] += a[i];
    }
    enc_norm(x, final_norm, n, h, c->eps, hidden_out);
    free(x); free(a); free(qkv); free(att); free(up); free(g);
}
