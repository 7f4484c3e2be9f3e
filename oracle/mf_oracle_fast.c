/*
 * mf_oracle_fast.c -- the timed CPU arm: one layer of batched paged decode (append + GQA
 * attention), same math as mfo_paged_decode_layer in mf_oracle.c, written for speed.
 *
 * TEST INFRASTRUCTURE ONLY (bench.py's cpu_baseline and reference arm, and the test that holds
 * it to the strict oracle).  The product never links it.
 *
 * The math is the reference's CPU oracle for this path (tests/sdpa_v2_parity.rs:37-133 of
 * cchance27/test-burn: q and the new k rounded to f16 after RoPE, f16 x f16 products
 * accumulated in f32, scores * scale, online softmax from -1e30, acc / l when |l| > 1e-6,
 * one rounding to f16) in the block order of the reference kernel (flash_decode.metal:188-317:
 * a block of keys, the block maximum, weights exp(score - block_max), one (m, l) update per
 * block).  What differs from the strict build is only what a competent CPU implementation
 * would change: K and V cross memory once per KV head and serve all G query heads of the
 * group, f16 -> f32 conversion uses F16C (vcvtph2ps) instead of a table, dot products and
 * the P*V update run on 8-wide FMA vectors, and the (sequence, kv head) units are spread
 * over all cores with OpenMP, longest first.  Reduction order therefore differs from the
 * strict oracle; tests hold the two within 2e-3.
 *
 * Build (on the machine that runs it, because of -march=native):
 *   gcc -O3 -march=native -fopenmp -fPIC -shared mf_oracle_fast.c -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#if defined(__AVX2__) && defined(__F16C__) && defined(__FMA__)
#include <immintrin.h>
#define MFO_FAST_SIMD 1
#else
#define MFO_FAST_SIMD 0
#endif

#define NEG_SENTINEL (-1e30f)
#define L_EPS 1e-6f
#define MAX_D 256
#define MAX_G 16
#define BLOCK_KEYS 16

int mfo_fast_simd(void) { return MFO_FAST_SIMD; }

int mfo_fast_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void mfo_fast_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* scalar binary16 conversions (IEEE round-to-nearest-even), used outside the hot loop */
static float h2f(uint16_t h)
{
#if MFO_FAST_SIMD
    return _cvtsh_ss(h);
#else
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do {
                man <<= 1;
                ++e;
            } while ((man & 0x400u) == 0);
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
#endif
}

static uint16_t f2h(float x)
{
#if MFO_FAST_SIMD
    return _cvtss_sh(x, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
#else
    uint32_t bits;
    memcpy(&bits, &x, 4);
    uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    uint32_t absb = bits & 0x7FFFFFFFu;
    if (absb >= 0x7F800000u) return (uint16_t)(sign | (absb > 0x7F800000u ? 0x7E00u : 0x7C00u));
    if (absb >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);
    if (absb < 0x33000001u) return sign;
    int32_t e = (int32_t)(absb >> 23) - 127;
    uint32_t man = (absb & 0x7FFFFFu) | 0x800000u, shift, half_exp;
    if (e < -14) {
        shift = (uint32_t)(13 + (-14 - e));
        half_exp = 0;
    } else {
        shift = 13;
        half_exp = (uint32_t)(e + 15);
    }
    uint32_t q = man >> shift, rem = man & ((1u << shift) - 1u), halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) ++q;
    return (uint16_t)(sign | (half_exp == 0 ? q : ((half_exp - 1) << 10) + q));
#endif
}

/* kv_prep_fused.metal:66-82: element hd of a row after RoPE, rounded to f16.  The products are
 * exact in f32 (11 x 11 bit significands), so an FMA gives the same bits as two rounded operations. */
static uint16_t rope_elem(const uint16_t *x, const uint16_t *c_row, const uint16_t *s_row, uint32_t hd, uint32_t D,
                          uint32_t rope_mode)
{
    const uint32_t half = D >> 1;
    uint32_t pair, mate;
    int first;
    if (rope_mode == 0) {
        first = hd < half;
        pair = first ? hd : hd - half;
        mate = first ? hd + half : hd - half;
    } else {
        first = (hd & 1u) == 0;
        pair = hd >> 1;
        mate = hd ^ 1u;
    }
    const float c = h2f(c_row[pair]), s = h2f(s_row[pair]);
    const float xi = first ? h2f(x[hd]) : h2f(x[mate]), xj = first ? h2f(x[mate]) : h2f(x[hd]);
    const float a = first ? xi * c : xj * c, b = first ? xj * s : xi * s;  /* exact products: contraction changes nothing */
    return f2h(first ? a - b : a + b);
}

/* One block of n <= BLOCK_KEYS consecutive rows of one kv head (k_rows / v_rows are n x D f16,
 * contiguous): scores for the G heads, block maximum, weights, (m, l, acc) update. */
static void block_update(const uint16_t *k_rows, const uint16_t *v_rows, uint32_t n, uint32_t D, uint32_t G,
                         const float *qf /* [G][D] */, float scale, float *m, float *l, float *acc /* [G][D] */)
{
    float s[MAX_G][BLOCK_KEYS];
#if MFO_FAST_SIMD
    for (uint32_t j = 0; j < n; ++j) {
        __m256 kv[MAX_D / 8];
        for (uint32_t c = 0; c < D / 8; ++c) kv[c] = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *)(k_rows + (size_t)j * D + 8 * c)));
        for (uint32_t g = 0; g < G; ++g) {
            __m256 a0 = _mm256_setzero_ps(), a1 = _mm256_setzero_ps();
            const float *qg = qf + (size_t)g * D;
            for (uint32_t c = 0; c < D / 8; c += 2) {
                a0 = _mm256_fmadd_ps(kv[c], _mm256_loadu_ps(qg + 8 * c), a0);
                a1 = _mm256_fmadd_ps(kv[c + 1], _mm256_loadu_ps(qg + 8 * c + 8), a1);
            }
            a0 = _mm256_add_ps(a0, a1);
            __m128 r = _mm_add_ps(_mm256_castps256_ps128(a0), _mm256_extractf128_ps(a0, 1));
            r = _mm_add_ps(r, _mm_movehl_ps(r, r));
            r = _mm_add_ss(r, _mm_shuffle_ps(r, r, 1));
            float sc = _mm_cvtss_f32(r) * scale;
            if (!isfinite(sc)) sc = NEG_SENTINEL;
            s[g][j] = sc;
        }
    }
#else
    for (uint32_t j = 0; j < n; ++j) {
        float kf[MAX_D];
        for (uint32_t d = 0; d < D; ++d) kf[d] = h2f(k_rows[(size_t)j * D + d]);
        for (uint32_t g = 0; g < G; ++g) {
            float a = 0.f;
            for (uint32_t d = 0; d < D; ++d) a += kf[d] * qf[(size_t)g * D + d];
            float sc = a * scale;
            if (!isfinite(sc)) sc = NEG_SENTINEL;
            s[g][j] = sc;
        }
    }
#endif
    float w[MAX_G][BLOCK_KEYS], alpha[MAX_G];
    for (uint32_t g = 0; g < G; ++g) {
        float bm = NEG_SENTINEL;
        for (uint32_t j = 0; j < n; ++j) bm = s[g][j] > bm ? s[g][j] : bm;
        const float mn = m[g] > bm ? m[g] : bm;
        float sum = 0.f;
        for (uint32_t j = 0; j < n; ++j) {
            w[g][j] = expf(s[g][j] - mn);
            sum += w[g][j];
        }
        alpha[g] = expf(m[g] - mn);
        l[g] = l[g] * alpha[g] + sum;
        m[g] = mn;
    }
#if MFO_FAST_SIMD
    for (uint32_t g = 0; g < G; ++g) {
        float *ag = acc + (size_t)g * D;
        const __m256 al = _mm256_set1_ps(alpha[g]);
        for (uint32_t c = 0; c < D / 8; ++c) _mm256_storeu_ps(ag + 8 * c, _mm256_mul_ps(_mm256_loadu_ps(ag + 8 * c), al));
    }
    for (uint32_t j = 0; j < n; ++j) {
        __m256 vv[MAX_D / 8];
        for (uint32_t c = 0; c < D / 8; ++c) vv[c] = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *)(v_rows + (size_t)j * D + 8 * c)));
        for (uint32_t g = 0; g < G; ++g) {
            float *ag = acc + (size_t)g * D;
            const __m256 wj = _mm256_set1_ps(w[g][j]);
            for (uint32_t c = 0; c < D / 8; ++c) _mm256_storeu_ps(ag + 8 * c, _mm256_fmadd_ps(vv[c], wj, _mm256_loadu_ps(ag + 8 * c)));
        }
    }
#else
    for (uint32_t g = 0; g < G; ++g)
        for (uint32_t d = 0; d < D; ++d) acc[(size_t)g * D + d] *= alpha[g];
    for (uint32_t j = 0; j < n; ++j)
        for (uint32_t g = 0; g < G; ++g)
            for (uint32_t d = 0; d < D; ++d) acc[(size_t)g * D + d] += w[g][j] * h2f(v_rows[(size_t)j * D + d]);
#endif
}

/* Same signature and result layout as mfo_paged_decode_layer (mf_oracle.h).  Requires
 * head_dim % 16 == 0, head_dim <= 256, group <= 16; returns -1 otherwise (nothing is computed). */
int mfo_fast_paged_decode_layer(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint16_t *k_pool,
                                uint16_t *v_pool, const uint16_t *cos_t, const uint16_t *sin_t,
                                const uint32_t *page_table, uint32_t pt_stride, const uint32_t *kv_lens, uint32_t batch,
                                uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint32_t page_size,
                                uint32_t rope_mode, float scale, uint16_t *out)
{
    const uint32_t D = head_dim, half = D >> 1, G = n_heads / n_kv_heads;
    if (D % 16 || D > MAX_D || G == 0 || G > MAX_G || page_size == 0) return -1;
    /* units, longest sequence first, so that the dynamic schedule ends evenly */
    const uint32_t n_units = batch * n_kv_heads;
    uint32_t *order = (uint32_t *)malloc(sizeof(uint32_t) * (batch ? batch : 1));
    for (uint32_t b = 0; b < batch; ++b) order[b] = b;
    for (uint32_t i = 1; i < batch; ++i) { /* insertion sort: batch is small */
        uint32_t x = order[i], j = i;
        while (j > 0 && kv_lens[order[j - 1]] < kv_lens[x]) {
            order[j] = order[j - 1];
            --j;
        }
        order[j] = x;
    }
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 1)
#endif
    for (uint32_t u = 0; u < n_units; ++u) {
        const uint32_t b = order[u / n_kv_heads], kh = u % n_kv_heads;
        const uint32_t L = kv_lens[b];
        if (L == 0) continue;
        const uint32_t pos = L - 1;
        const uint32_t *pt = page_table + (size_t)b * pt_stride;
        const uint16_t *c_row = cos_t + (size_t)pos * half, *s_row = sin_t + (size_t)pos * half;
        {
            const uint16_t *ks = k + ((size_t)b * n_kv_heads + kh) * D, *vs = v + ((size_t)b * n_kv_heads + kh) * D;
            const size_t slot = (((size_t)pt[pos / page_size] * n_kv_heads + kh) * page_size + pos % page_size) * D;
            for (uint32_t hd = 0; hd < D; ++hd) k_pool[slot + hd] = rope_elem(ks, c_row, s_row, hd, D, rope_mode);
            memcpy(v_pool + slot, vs, (size_t)D * 2);
        }
        float qf[MAX_G * MAX_D], acc[MAX_G * MAX_D], m[MAX_G], l[MAX_G];
        for (uint32_t g = 0; g < G; ++g) {
            const uint16_t *src = q + ((size_t)b * n_heads + kh * G + g) * D;
            for (uint32_t hd = 0; hd < D; ++hd) qf[(size_t)g * D + hd] = h2f(rope_elem(src, c_row, s_row, hd, D, rope_mode));
            m[g] = NEG_SENTINEL;
            l[g] = 0.f;
        }
        memset(acc, 0, sizeof(float) * (size_t)G * D);
        for (uint32_t t0 = 0; t0 < L;) {
            /* rows of one page are contiguous for a kv head: walk page by page, BLOCK_KEYS rows at a time */
            const uint32_t in_page = t0 % page_size;
            uint32_t n = page_size - in_page;
            if (n > BLOCK_KEYS) n = BLOCK_KEYS;
            if (n > L - t0) n = L - t0;
            const size_t row = (((size_t)pt[t0 / page_size] * n_kv_heads + kh) * page_size + in_page) * D;
            block_update(k_pool + row, v_pool + row, n, D, G, qf, scale, m, l, acc);
            t0 += n;
        }
        for (uint32_t g = 0; g < G; ++g) {
            uint16_t *dst = out + ((size_t)b * n_heads + kh * G + g) * D;
            const int ok = isfinite(l[g]) && fabsf(l[g]) > L_EPS;
            for (uint32_t d = 0; d < D; ++d) {
                float r = ok ? acc[(size_t)g * D + d] / l[g] : acc[(size_t)g * D + d];
                if (!isfinite(r)) r = 0.f;
                dst[d] = f2h(r);
            }
        }
    }
    free(order);
    return 0;
}
