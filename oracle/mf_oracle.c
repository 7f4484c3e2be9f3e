/*
 * mf_oracle.c -- CPU restatement of the metallic-foundry KV-cache hot path.
 * TEST INFRASTRUCTURE ONLY; see mf_oracle.h for provenance and pin status.
 *
 * Build: gcc -O2 -ffp-contract=off -fPIC -shared [-fopenmp] mf_oracle.c -lm
 * (-ffp-contract=off keeps every f32 operation a separately rounded IEEE op, so
 * results do not depend on whether the host CPU has FMA).
 */
#include "mf_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define MFO_NEG_SENTINEL (-1e30f) /* streaming.metal:27, flash_decode.metal:173 */
#define MFO_L_EPS 1e-6f           /* flash_decode.metal:308, flash_prefill.metal:258 */

/* ------------------------------------------------------------------ f16 --- */

float mfo_f16_to_f32(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: renormalise */
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
}

uint16_t mfo_f32_to_f16(float x)
{
    uint32_t bits;
    memcpy(&bits, &x, 4);
    uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    uint32_t absb = bits & 0x7FFFFFFFu;
    if (absb >= 0x7F800000u) { /* inf / nan */
        if (absb > 0x7F800000u) return (uint16_t)(sign | 0x7E00u | ((absb >> 13) & 0x3FFu));
        return (uint16_t)(sign | 0x7C00u);
    }
    if (absb >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to inf */
    if (absb < 0x33000001u) return sign;                         /* <= 2^-25 -> 0 */
    int32_t e = (int32_t)(absb >> 23) - 127;
    uint32_t man = (absb & 0x7FFFFFu) | 0x800000u; /* 24-bit significand */
    uint32_t shift, half_exp;
    if (e < -14) { /* subnormal result */
        shift = (uint32_t)(13 + (-14 - e));
        half_exp = 0;
    } else {
        shift = 13;
        half_exp = (uint32_t)(e + 15);
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) ++q;
    uint32_t out;
    if (half_exp == 0) {
        out = q; /* may carry into the exponent field, which is the right result */
    } else {
        out = ((half_exp - 1) << 10) + q; /* q carries the implicit 1 (0x400) */
    }
    return (uint16_t)(sign | out);
}

static float g_h2f[65536];
static int g_h2f_ready = 0;

static void h2f_init(void)
{
    if (g_h2f_ready) return;
#ifdef _OPENMP
#pragma omp critical(mfo_h2f)
#endif
    {
        if (!g_h2f_ready) {
            for (uint32_t i = 0; i < 65536u; ++i) g_h2f[i] = mfo_f16_to_f32((uint16_t)i);
            g_h2f_ready = 1;
        }
    }
}
#define H2F(h) (g_h2f[(h)])

/* ------------------------------------------------------------ generators --- */

uint32_t mfo_lcg_fill_f16(uint32_t state, uint16_t *out, size_t n, float scale)
{
    for (size_t i = 0; i < n; ++i) {
        state = state * 1664525u + 1013904223u;
        float r01 = (float)(state >> 9) * (1.0f / (float)(1u << 23));
        out[i] = mfo_f32_to_f16((r01 * 2.0f - 1.0f) * scale);
    }
    return state;
}

uint64_t mfo_splitmix64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

void mfo_normal_fill_f16(uint64_t seed, uint64_t tensor_id, uint64_t first, uint16_t *out,
                         size_t n)
{
    const uint64_t stream = seed ^ (tensor_id * 0x9E3779B97F4A7C15ull);
    for (size_t i = 0; i < n; ++i) {
        uint64_t r = mfo_splitmix64(stream ^ (first + i));
        /* two 32-bit halves -> u1 in (0,1], u2 in [0,1) */
        double u1 = ((double)(uint32_t)(r >> 32) + 1.0) * (1.0 / 4294967296.0);
        double u2 = (double)(uint32_t)r * (1.0 / 4294967296.0);
        double z = sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925 * u2);
        out[i] = mfo_f32_to_f16((float)z);
    }
}

/* ------------------------------------------------------------ RoPE tables --- */

void mfo_rope_tables(float theta, uint32_t head_dim, uint32_t first_pos, uint32_t n_pos,
                     const float *freq_factors, uint16_t *cos_out, uint16_t *sin_out)
{
    const uint32_t half = head_dim / 2;
    float *inv = (float *)malloc(sizeof(float) * (half ? half : 1));
    for (uint32_t i = 0; i < half; ++i) {
        float exponent = (float)(2 * i) / (float)head_dim;
        float f = 1.0f / powf(theta, exponent);
        if (freq_factors) f /= freq_factors[i];
        inv[i] = f;
    }
    for (uint32_t r = 0; r < n_pos; ++r) {
        float p = (float)(first_pos + r);
        for (uint32_t i = 0; i < half; ++i) {
            float angle = p * inv[i];
            cos_out[(size_t)r * half + i] = mfo_f32_to_f16(cosf(angle));
            sin_out[(size_t)r * half + i] = mfo_f32_to_f16(sinf(angle));
        }
    }
    free(inv);
}

/* ---------------------------------------------------------- unfused chain --- */

void mfo_rope_neox(const uint16_t *in, uint16_t *out, const uint16_t *cos_t,
                   const uint16_t *sin_t, uint32_t dim, uint32_t seq_len,
                   uint32_t position_offset, size_t total_elements)
{
    h2f_init();
    const uint32_t half = dim / 2;
    for (size_t gid = 0; gid < total_elements; ++gid) {
        uint32_t f = (uint32_t)(gid % dim);
        size_t row = gid / dim;
        size_t pos = (row % seq_len) + position_offset;
        uint32_t pair = f < half ? f : f - half;
        float c = H2F(cos_t[pos * half + pair]);
        float s = H2F(sin_t[pos * half + pair]);
        float r;
        if (f < half) {
            float xi = H2F(in[gid]);
            float xj = H2F(in[row * dim + f + half]);
            r = xi * c - xj * s;
        } else {
            float xj = H2F(in[gid]);
            float xi = H2F(in[row * dim + (f - half)]);
            r = xj * c + xi * s;
        }
        out[gid] = mfo_f32_to_f16(r);
    }
}

void mfo_kv_rearrange(const uint16_t *in, uint16_t *out, uint32_t row_stride,
                      uint32_t kv_head_dim, uint32_t n_heads, uint32_t n_kv_heads,
                      uint32_t head_dim, uint32_t seq)
{
    const uint32_t group = n_heads / n_kv_heads;
    for (uint32_t h = 0; h < n_heads; ++h)
        for (uint32_t s = 0; s < seq; ++s)
            for (uint32_t d = 0; d < head_dim; ++d) {
                uint32_t src_h = h / group;
                size_t src = (size_t)s * row_stride + (size_t)src_h * kv_head_dim + d;
                out[((size_t)h * seq + s) * head_dim + d] = in[src];
            }
}

void mfo_kv_cache_write(uint16_t *cache, const uint16_t *in, uint32_t n_kv_heads,
                        uint32_t head_dim, uint32_t input_seq_len, uint32_t position_offset,
                        uint32_t max_seq_len)
{
    for (uint32_t h = 0; h < n_kv_heads; ++h)
        for (uint32_t s = 0; s < input_seq_len; ++s)
            memcpy(cache + ((size_t)h * max_seq_len + position_offset + s) * head_dim,
                   in + ((size_t)h * input_seq_len + s) * head_dim, (size_t)head_dim * 2);
}

void mfo_kv_cache_write_repeat(uint16_t *cache, const uint16_t *in, uint32_t n_kv_heads,
                               uint32_t group_size, uint32_t head_dim, uint32_t input_seq_len,
                               uint32_t position_offset, uint32_t max_seq_len)
{
    for (uint32_t h = 0; h < n_kv_heads; ++h)
        for (uint32_t g = 0; g < group_size; ++g)
            for (uint32_t s = 0; s < input_seq_len; ++s)
                memcpy(cache + ((size_t)(h * group_size + g) * max_seq_len + position_offset + s) *
                                   head_dim,
                       in + ((size_t)h * input_seq_len + s) * head_dim, (size_t)head_dim * 2);
}

void mfo_kv_cache_read(const uint16_t *cache, uint16_t *out, uint32_t n_kv_heads,
                       uint32_t head_dim, uint32_t seq_len, uint32_t max_seq_len)
{
    for (uint32_t h = 0; h < n_kv_heads; ++h)
        memcpy(out + (size_t)h * seq_len * head_dim, cache + (size_t)h * max_seq_len * head_dim,
               (size_t)seq_len * head_dim * 2);
}

void mfo_kv_cache_grow(const uint16_t *old_cache, uint16_t *new_cache, uint32_t heads, uint32_t head_dim,
                       uint32_t old_capacity, uint32_t new_capacity, uint32_t current_pos)
{
    /* src/model/executor.rs:2493-2504: one copy of current_pos*head_dim*2 bytes per head */
    for (uint32_t h = 0; h < heads; ++h)
        memcpy(new_cache + (size_t)h * new_capacity * head_dim, old_cache + (size_t)h * old_capacity * head_dim,
               (size_t)current_pos * head_dim * 2);
}

void mfo_paged_scatter(const uint16_t *cache, uint16_t *pool, const uint32_t *page_table_row, uint32_t L,
                       uint32_t n_kv_heads, uint32_t capacity, uint32_t page_size, uint32_t head_dim)
{
    for (uint32_t kh = 0; kh < n_kv_heads; ++kh)
        for (uint32_t t = 0; t < L; ++t) {
            uint32_t page = page_table_row[t / page_size];
            size_t dst = (((size_t)page * n_kv_heads + kh) * page_size + t % page_size) * head_dim;
            memcpy(pool + dst, cache + ((size_t)kh * capacity + t) * head_dim, (size_t)head_dim * 2);
        }
}

void mfo_repeat_kv_heads(const uint16_t *in, uint16_t *out, uint32_t n_kv_heads,
                         uint32_t group_size, uint32_t seq, uint32_t head_dim)
{
    for (uint32_t h = 0; h < n_kv_heads * group_size; ++h)
        memcpy(out + (size_t)h * seq * head_dim, in + (size_t)(h / group_size) * seq * head_dim,
               (size_t)seq * head_dim * 2);
}

/* ------------------------------------------------------------ fused append --- */

/* One roped element of a head row `x` (length D) at table row (c_row, s_row).
 * kv_prep_fused.metal:60-83. */
static inline uint16_t rope_elem(const uint16_t *x, const uint16_t *c_row, const uint16_t *s_row,
                                 uint32_t hd, uint32_t head_dim, uint32_t rope_mode)
{
    const uint32_t half = head_dim >> 1;
    const int normal = rope_mode == 1;
    uint32_t pair = normal ? (hd >> 1) : (hd < half ? hd : hd - half);
    int first = normal ? ((hd & 1u) == 0) : (hd < half);
    uint32_t mate = normal ? (first ? hd + 1 : hd - 1) : (first ? hd + half : hd - half);
    float c = H2F(c_row[pair]);
    float s = H2F(s_row[pair]);
    float r;
    if (first) {
        float xi = H2F(x[hd]), xj = H2F(x[mate]);
        r = xi * c - xj * s;
    } else {
        float xj = H2F(x[hd]), xi = H2F(x[mate]);
        r = xj * c + xi * s;
    }
    return mfo_f32_to_f16(r);
}

static void project_rows(const uint16_t *xn, const uint16_t *w, const uint16_t *bias, uint32_t k_dim,
                         uint32_t n, uint32_t wpb, uint16_t *out)
{
    for (uint32_t r = 0; r < n; ++r) {
        float acc = 0.0f;
        for (uint32_t k = 0; k < k_dim; ++k) {
            size_t idx = wpb ? (size_t)(k % wpb) + (size_t)wpb * (r + (size_t)(k / wpb) * n)
                             : (size_t)r * k_dim + k;
            acc += H2F(xn[k]) * H2F(w[idx]);
        }
        out[r] = mfo_f32_to_f16(acc + (bias ? H2F(bias[r]) : 0.0f));
    }
}

void mfo_fused_qkv(const uint16_t *input, const uint16_t *w_q, const uint16_t *w_k,
                   const uint16_t *w_v, const uint16_t *gamma, const uint16_t *b_q,
                   const uint16_t *b_k, const uint16_t *b_v, uint32_t m, uint32_t k_dim,
                   uint32_t n_dim, uint32_t n_kv, uint32_t weights_per_block, float eps,
                   uint16_t *out_q, uint16_t *out_k, uint16_t *out_v)
{
    h2f_init();
    uint16_t *xn = (uint16_t *)malloc((size_t)k_dim * sizeof(uint16_t));
    for (uint32_t row = 0; row < m; ++row) {
        const uint16_t *x = input + (size_t)row * k_dim;
        if (gamma) {
            float sum_sq = 0.0f;
            for (uint32_t k = 0; k < k_dim; ++k) sum_sq += H2F(x[k]) * H2F(x[k]);
            const float inv_rms = 1.0f / sqrtf(sum_sq / (float)k_dim + eps);
            for (uint32_t k = 0; k < k_dim; ++k) xn[k] = mfo_f32_to_f16((H2F(x[k]) * inv_rms) * H2F(gamma[k]));
        } else {
            memcpy(xn, x, (size_t)k_dim * sizeof(uint16_t));
        }
        project_rows(xn, w_q, b_q, k_dim, n_dim, weights_per_block, out_q + (size_t)row * n_dim);
        project_rows(xn, w_k, b_k, k_dim, n_kv, weights_per_block, out_k + (size_t)row * n_kv);
        project_rows(xn, w_v, b_v, k_dim, n_kv, weights_per_block, out_v + (size_t)row * n_kv);
    }
    free(xn);
}

void mfo_kv_prep_fused(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint16_t *q_rot,
                       uint16_t *k_cache, uint16_t *v_cache, const uint16_t *cos_t,
                       const uint16_t *sin_t, const mfo_kv_prep_params *p, int expanded)
{
    h2f_init();
    const uint32_t D = p->head_dim, M = p->seq_len, half = D >> 1;
    const int apply =
        p->no_rope_layer_step == 0 || ((p->layer_idx + 1u) % p->no_rope_layer_step) != 0u;
    const size_t head_stride = (size_t)p->max_seq_len * D;
    for (uint32_t gid = 0; gid < p->total_elements; ++gid) {
        uint32_t hd = gid % D;
        uint32_t t = gid / D;
        uint32_t s = t % M;
        uint32_t h = t / M;
        uint32_t pos = p->position_offset + s;
        const uint16_t *c_row = cos_t + (size_t)pos * half;
        const uint16_t *s_row = sin_t + (size_t)pos * half;
        const uint16_t *q_head = q + (size_t)s * p->d_model + (size_t)h * D;
        q_rot[gid] = apply ? rope_elem(q_head, c_row, s_row, hd, D, p->rope_mode) : q_head[hd];
        if (h % p->group_size != 0) continue;
        uint32_t kv_h = h / p->group_size;
        const uint16_t *k_head = k + (size_t)s * p->kv_dim + (size_t)kv_h * D;
        const uint16_t *v_head = v + (size_t)s * p->kv_dim + (size_t)kv_h * D;
        uint16_t kr = apply ? rope_elem(k_head, c_row, s_row, hd, D, p->rope_mode) : k_head[hd];
        uint16_t vr = v_head[hd];
        if (!expanded) {
            size_t idx = (size_t)kv_h * head_stride + (size_t)pos * D + hd;
            k_cache[idx] = kr;
            v_cache[idx] = vr;
        } else {
            for (uint32_t g = 0; g < p->group_size; ++g) {
                size_t idx = (size_t)(kv_h * p->group_size + g) * head_stride + (size_t)pos * D + hd;
                k_cache[idx] = kr;
                v_cache[idx] = vr;
            }
        }
    }
}

void mfo_paged_kv_append(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint16_t *q_rot,
                         uint16_t *k_pool, uint16_t *v_pool, const uint16_t *cos_t,
                         const uint16_t *sin_t, const uint32_t *page_table, uint32_t pt_stride,
                         const uint32_t *positions, uint32_t batch, uint32_t n_heads,
                         uint32_t n_kv_heads, uint32_t head_dim, uint32_t page_size,
                         uint32_t rope_mode, int apply_rope)
{
    h2f_init();
    const uint32_t D = head_dim, half = D >> 1;
    for (uint32_t b = 0; b < batch; ++b) {
        uint32_t pos = positions[b];
        const uint16_t *c_row = cos_t + (size_t)pos * half;
        const uint16_t *s_row = sin_t + (size_t)pos * half;
        for (uint32_t h = 0; h < n_heads; ++h) {
            const uint16_t *src = q + ((size_t)b * n_heads + h) * D;
            uint16_t *dst = q_rot + ((size_t)b * n_heads + h) * D;
            for (uint32_t hd = 0; hd < D; ++hd)
                dst[hd] = apply_rope ? rope_elem(src, c_row, s_row, hd, D, rope_mode) : src[hd];
        }
        uint32_t page = page_table[(size_t)b * pt_stride + pos / page_size];
        uint32_t row = pos % page_size;
        for (uint32_t kh = 0; kh < n_kv_heads; ++kh) {
            const uint16_t *ks = k + ((size_t)b * n_kv_heads + kh) * D;
            const uint16_t *vs = v + ((size_t)b * n_kv_heads + kh) * D;
            size_t slot = (((size_t)page * n_kv_heads + kh) * page_size + row) * D;
            for (uint32_t hd = 0; hd < D; ++hd) {
                k_pool[slot + hd] = apply_rope ? rope_elem(ks, c_row, s_row, hd, D, rope_mode) : ks[hd];
                v_pool[slot + hd] = vs[hd];
            }
        }
    }
}

void mfo_paged_gather(const uint16_t *pool, const uint32_t *page_table_row, uint32_t L,
                      uint32_t n_kv_heads, uint32_t page_size, uint32_t head_dim, uint16_t *out)
{
    for (uint32_t kh = 0; kh < n_kv_heads; ++kh)
        for (uint32_t t = 0; t < L; ++t) {
            uint32_t page = page_table_row[t / page_size];
            size_t src = (((size_t)page * n_kv_heads + kh) * page_size + t % page_size) * head_dim;
            memcpy(out + ((size_t)kh * L + t) * head_dim, pool + src, (size_t)head_dim * 2);
        }
}

/* --------------------------------------------------------------- decode --- */

static inline float dot_f16(const uint16_t *a, const uint16_t *b, uint32_t n)
{
    float acc = 0.0f;
    for (uint32_t d = 0; d < n; ++d) acc += H2F(a[d]) * H2F(b[d]);
    return acc;
}

/* Online update for one key (tests/sdpa_v2_parity.rs:108-123). */
static inline void online_step(float score, const uint16_t *v_row, uint32_t D, float *m, float *l,
                               float *acc)
{
    float m_new = *m > score ? *m : score;
    float w = expf(score - m_new);
    float a = expf(*m - m_new);
    *l = *l * a + w;
    *m = m_new;
    for (uint32_t d = 0; d < D; ++d) acc[d] = acc[d] * a + H2F(v_row[d]) * w;
}

static inline void finish_decode_row(const float *acc, float l, uint32_t D, uint16_t *out)
{
    /* flash_decode.metal:306-317: divide when l is finite and |l| > 1e-6,
     * else leave unscaled; non-finite results become 0. */
    int ok = isfinite(l) && fabsf(l) > MFO_L_EPS;
    for (uint32_t d = 0; d < D; ++d) {
        float r = ok ? acc[d] / l : acc[d];
        if (!isfinite(r)) r = 0.0f;
        out[d] = mfo_f32_to_f16(r);
    }
}

void mfo_decode_online(const uint16_t *q_rot, const uint16_t *k_cache, const uint16_t *v_cache,
                       uint32_t n_heads, uint32_t cache_heads, uint32_t head_dim,
                       uint32_t capacity, uint32_t key_begin, uint32_t key_end, float scale,
                       uint16_t *out, float *acc_out, float *m_out, float *l_out)
{
    h2f_init();
    const uint32_t D = head_dim;
    uint32_t group = n_heads / (cache_heads ? cache_heads : 1);
    if (group == 0) group = 1;
    float *acc = (float *)malloc(sizeof(float) * D);
    for (uint32_t h = 0; h < n_heads; ++h) {
        uint32_t kvh = h / group;
        const uint16_t *qh = q_rot + (size_t)h * D;
        const uint16_t *kb = k_cache + (size_t)kvh * capacity * D;
        const uint16_t *vb = v_cache + (size_t)kvh * capacity * D;
        float m = MFO_NEG_SENTINEL, l = 0.0f;
        for (uint32_t d = 0; d < D; ++d) acc[d] = 0.0f;
        for (uint32_t t = key_begin; t < key_end; ++t) {
            float score = dot_f16(qh, kb + (size_t)t * D, D) * scale;
            if (!isfinite(score)) score = MFO_NEG_SENTINEL; /* flash_decode.metal:214-216 */
            online_step(score, vb + (size_t)t * D, D, &m, &l, acc);
        }
        if (out) finish_decode_row(acc, l, D, out + (size_t)h * D);
        if (acc_out) memcpy(acc_out + (size_t)h * D, acc, sizeof(float) * D);
        if (m_out) m_out[h] = m;
        if (l_out) l_out[h] = l;
    }
    free(acc);
}

void mfo_decode_blocked(const uint16_t *q_rot, const uint16_t *k_cache, const uint16_t *v_cache,
                        uint32_t n_heads, uint32_t cache_heads, uint32_t head_dim,
                        uint32_t capacity, uint32_t kv_len, uint32_t block_keys, float scale,
                        uint16_t *out)
{
    h2f_init();
    const uint32_t D = head_dim;
    uint32_t group = n_heads / (cache_heads ? cache_heads : 1);
    if (group == 0) group = 1;
    if (kv_len == 0) return; /* flash_decode.metal:168: nothing is written */
    float *acc = (float *)malloc(sizeof(float) * D * 2);
    float *blk = acc + D;
    float *scores = (float *)malloc(sizeof(float) * block_keys);
    for (uint32_t h = 0; h < n_heads; ++h) {
        uint32_t kvh = h / group;
        const uint16_t *qh = q_rot + (size_t)h * D;
        const uint16_t *kb = k_cache + (size_t)kvh * capacity * D;
        const uint16_t *vb = v_cache + (size_t)kvh * capacity * D;
        float m = MFO_NEG_SENTINEL, l = 0.0f;
        for (uint32_t d = 0; d < D; ++d) acc[d] = 0.0f;
        for (uint32_t base = 0; base < kv_len; base += block_keys) {
            uint32_t n = kv_len - base < block_keys ? kv_len - base : block_keys;
            float bm = MFO_NEG_SENTINEL;
            for (uint32_t j = 0; j < n; ++j) {
                float s = dot_f16(qh, kb + (size_t)(base + j) * D, D) * scale;
                if (!isfinite(s)) s = MFO_NEG_SENTINEL;
                scores[j] = s;
                if (s > bm) bm = s;
            }
            float bsum = 0.0f;
            for (uint32_t d = 0; d < D; ++d) blk[d] = 0.0f;
            for (uint32_t j = 0; j < n; ++j) {
                float w = expf(scores[j] - bm);
                bsum += w;
                const uint16_t *vr = vb + (size_t)(base + j) * D;
                for (uint32_t d = 0; d < D; ++d) blk[d] += H2F(vr[d]) * w;
            }
            float m_new = m > bm ? m : bm;
            float alpha = expf(m - m_new), beta = expf(bm - m_new);
            l = l * alpha + bsum * beta;
            m = m_new;
            for (uint32_t d = 0; d < D; ++d) acc[d] = acc[d] * alpha + blk[d] * beta;
        }
        finish_decode_row(acc, l, D, out + (size_t)h * D);
    }
    free(scores);
    free(acc);
}

void mfo_decode_gold(const uint16_t *q_rot, const uint16_t *k_cache, const uint16_t *v_cache,
                     uint32_t n_heads, uint32_t cache_heads, uint32_t head_dim, uint32_t capacity,
                     uint32_t kv_len, float scale, double *out)
{
    h2f_init();
    const uint32_t D = head_dim;
    uint32_t group = n_heads / (cache_heads ? cache_heads : 1);
    if (group == 0) group = 1;
    double *sc = (double *)malloc(sizeof(double) * (kv_len ? kv_len : 1));
    for (uint32_t h = 0; h < n_heads; ++h) {
        uint32_t kvh = h / group;
        const uint16_t *qh = q_rot + (size_t)h * D;
        const uint16_t *kb = k_cache + (size_t)kvh * capacity * D;
        const uint16_t *vb = v_cache + (size_t)kvh * capacity * D;
        double mx = -INFINITY;
        for (uint32_t t = 0; t < kv_len; ++t) {
            double a = 0.0;
            for (uint32_t d = 0; d < D; ++d) a += (double)H2F(qh[d]) * (double)H2F(kb[(size_t)t * D + d]);
            sc[t] = a * (double)scale;
            if (sc[t] > mx) mx = sc[t];
        }
        double den = 0.0;
        for (uint32_t t = 0; t < kv_len; ++t) {
            sc[t] = exp(sc[t] - mx);
            den += sc[t];
        }
        for (uint32_t d = 0; d < D; ++d) {
            double a = 0.0;
            for (uint32_t t = 0; t < kv_len; ++t) a += sc[t] * (double)H2F(vb[(size_t)t * D + d]);
            out[(size_t)h * D + d] = den > 0.0 ? a / den : 0.0;
        }
    }
    free(sc);
}

void mfo_cpu_sdpa_attention(const uint16_t *q, const uint16_t *k, const uint16_t *v,
                            const uint16_t *cos_t, const uint16_t *sin_t, uint32_t batch_heads,
                            uint32_t kv_len, uint32_t head_dim, uint16_t *out)
{
    h2f_init();
    const uint32_t D = head_dim, half = D / 2;
    const float scale = 1.0f / sqrtf((float)D);
    const uint32_t q_pos = kv_len - 1;
    uint16_t *qr = (uint16_t *)malloc((size_t)batch_heads * D * 2);
    uint16_t *kr = (uint16_t *)malloc((size_t)batch_heads * kv_len * D * 2);
    for (uint32_t b = 0; b < batch_heads; ++b) {
        for (uint32_t i = 0; i < half; ++i) {
            float c = H2F(cos_t[(size_t)q_pos * half + i]), s = H2F(sin_t[(size_t)q_pos * half + i]);
            float x0 = H2F(q[(size_t)b * D + i]), x1 = H2F(q[(size_t)b * D + half + i]);
            qr[(size_t)b * D + i] = mfo_f32_to_f16(x0 * c - x1 * s);
            qr[(size_t)b * D + half + i] = mfo_f32_to_f16(x0 * s + x1 * c);
        }
        for (uint32_t t = 0; t < kv_len; ++t) {
            size_t o = ((size_t)b * kv_len + t) * D;
            for (uint32_t i = 0; i < half; ++i) {
                float c = H2F(cos_t[(size_t)t * half + i]), s = H2F(sin_t[(size_t)t * half + i]);
                float x0 = H2F(k[o + i]), x1 = H2F(k[o + half + i]);
                kr[o + i] = mfo_f32_to_f16(x0 * c - x1 * s);
                kr[o + half + i] = mfo_f32_to_f16(x0 * s + x1 * c);
            }
        }
    }
    float *acc = (float *)malloc(sizeof(float) * D);
    for (uint32_t b = 0; b < batch_heads; ++b) {
        float m = MFO_NEG_SENTINEL, l = 0.0f;
        for (uint32_t d = 0; d < D; ++d) acc[d] = 0.0f;
        for (uint32_t t = 0; t < kv_len; ++t) {
            size_t o = ((size_t)b * kv_len + t) * D;
            float score = dot_f16(qr + (size_t)b * D, kr + o, D) * scale;
            online_step(score, v + o, D, &m, &l, acc);
        }
        for (uint32_t d = 0; d < D; ++d) {
            float r = fabsf(l) > MFO_L_EPS ? acc[d] / l : acc[d];
            out[(size_t)b * D + d] = mfo_f32_to_f16(r);
        }
    }
    free(acc);
    free(kr);
    free(qr);
}

/* -------------------------------------------------------------- prefill --- */

void mfo_splitk_tile_range(uint32_t kv_len, uint32_t split_k, uint32_t split_id,
                           uint32_t *tile_begin, uint32_t *tile_end)
{
    uint32_t tiles = (kv_len + 31) / 32;
    uint32_t per = (tiles + split_k - 1) / split_k;
    uint32_t b = split_id * per;
    uint32_t e = b + per < tiles ? b + per : tiles;
    if (b > tiles) b = tiles;
    if (e < b) e = b;
    *tile_begin = b;
    *tile_end = e;
}

void mfo_prefill_causal(const uint16_t *q, const uint16_t *k_cache, const uint16_t *v_cache,
                        uint32_t n_heads, uint32_t cache_heads, uint32_t head_dim,
                        uint32_t capacity, uint32_t q_len, uint32_t kv_len, uint32_t query_offset,
                        float scale, uint32_t tile_begin, uint32_t tile_end, uint16_t *out,
                        float *acc_out, float *m_out, float *l_out)
{
    h2f_init();
    const uint32_t D = head_dim;
    uint32_t group = n_heads / (cache_heads ? cache_heads : 1);
    if (group == 0) group = 1;
    const uint32_t tiles = (kv_len + 31) / 32;
    if (tile_end > tiles) tile_end = tiles;
#ifdef _OPENMP
#pragma omp parallel for collapse(2) schedule(dynamic, 8)
#endif
    for (uint32_t h = 0; h < n_heads; ++h) {
        for (uint32_t r = 0; r < q_len; ++r) {
            float acc[256], blk[256], sc[32];
            uint32_t kvh = h / group;
            const uint16_t *qh = q + ((size_t)h * q_len + r) * D;
            const uint16_t *kb = k_cache + (size_t)kvh * capacity * D;
            const uint16_t *vb = v_cache + (size_t)kvh * capacity * D;
            const uint32_t limit = r + query_offset; /* flash_prefill.metal:181 */
            float m = MFO_NEG_SENTINEL, l = 0.0f;
            for (uint32_t d = 0; d < D; ++d) acc[d] = 0.0f;
            for (uint32_t tile = tile_begin; tile < tile_end; ++tile) {
                uint32_t k0 = tile * 32;
                float bm = MFO_NEG_SENTINEL;
                uint32_t n = 0;
                for (uint32_t j = 0; j < 32 && k0 + j < kv_len; ++j, ++n) {
                    uint32_t kg = k0 + j;
                    float s = kg > limit ? MFO_NEG_SENTINEL : dot_f16(qh, kb + (size_t)kg * D, D) * scale;
                    sc[j] = s;
                    if (s > bm) bm = s;
                }
                float bsum = 0.0f;
                for (uint32_t d = 0; d < D; ++d) blk[d] = 0.0f;
                for (uint32_t j = 0; j < n; ++j) {
                    uint32_t kg = k0 + j;
                    if (kg > limit) continue;
                    float p = expf(sc[j] - bm);
                    bsum += p;
                    const uint16_t *vr = vb + (size_t)kg * D;
                    for (uint32_t d = 0; d < D; ++d) blk[d] += p * H2F(vr[d]);
                }
                float m_new = m > bm ? m : bm;
                float alpha = expf(m - m_new), beta = expf(bm - m_new);
                l = l * alpha + bsum * beta;
                m = m_new;
                for (uint32_t d = 0; d < D; ++d) acc[d] = acc[d] * alpha + blk[d] * beta;
            }
            if (acc_out) {
                memcpy(acc_out + ((size_t)h * q_len + r) * D, acc, sizeof(float) * D);
                m_out[(size_t)h * q_len + r] = m;
                l_out[(size_t)h * q_len + r] = l;
            }
            if (out) {
                float inv = (isfinite(l) && fabsf(l) > MFO_L_EPS) ? 1.0f / l : 0.0f;
                uint16_t *o = out + (size_t)r * n_heads * D + (size_t)h * D;
                for (uint32_t d = 0; d < D; ++d) o[d] = mfo_f32_to_f16(acc[d] * inv);
            }
        }
    }
}

void mfo_prefill_gold(const uint16_t *q, const uint16_t *k_cache, const uint16_t *v_cache,
                      uint32_t n_heads, uint32_t cache_heads, uint32_t head_dim, uint32_t capacity,
                      uint32_t q_len, uint32_t kv_len, uint32_t query_offset, float scale,
                      double *out)
{
    h2f_init();
    const uint32_t D = head_dim;
    uint32_t group = n_heads / (cache_heads ? cache_heads : 1);
    if (group == 0) group = 1;
#ifdef _OPENMP
#pragma omp parallel for collapse(2) schedule(dynamic, 8)
#endif
    for (uint32_t h = 0; h < n_heads; ++h) {
        for (uint32_t r = 0; r < q_len; ++r) {
            uint32_t kvh = h / group;
            const uint16_t *qh = q + ((size_t)h * q_len + r) * D;
            const uint16_t *kb = k_cache + (size_t)kvh * capacity * D;
            const uint16_t *vb = v_cache + (size_t)kvh * capacity * D;
            uint32_t vis = r + query_offset + 1;
            if (vis > kv_len) vis = kv_len;
            double *sc = (double *)malloc(sizeof(double) * (vis ? vis : 1));
            double mx = -INFINITY;
            for (uint32_t t = 0; t < vis; ++t) {
                double a = 0.0;
                for (uint32_t d = 0; d < D; ++d)
                    a += (double)H2F(qh[d]) * (double)H2F(kb[(size_t)t * D + d]);
                sc[t] = a * (double)scale;
                if (sc[t] > mx) mx = sc[t];
            }
            double den = 0.0;
            for (uint32_t t = 0; t < vis; ++t) {
                sc[t] = exp(sc[t] - mx);
                den += sc[t];
            }
            double *o = out + (size_t)r * n_heads * D + (size_t)h * D;
            for (uint32_t d = 0; d < D; ++d) {
                double a = 0.0;
                for (uint32_t t = 0; t < vis; ++t) a += sc[t] * (double)H2F(vb[(size_t)t * D + d]);
                o[d] = den > 0.0 ? a / den : 0.0;
            }
            free(sc);
        }
    }
}

/* ---------------------------------------------------------------- merge --- */

void mfo_merge_partials(const float *acc, const float *m, const float *l, uint32_t n_splits,
                        uint32_t rows, uint32_t head_dim, uint16_t *out)
{
    const uint32_t D = head_dim;
    for (uint32_t r = 0; r < rows; ++r) {
        float mx = MFO_NEG_SENTINEL;
        for (uint32_t s = 0; s < n_splits; ++s) {
            float ms = m[(size_t)s * rows + r];
            if (ms > mx) mx = ms;
        }
        float lt = 0.0f;
        for (uint32_t s = 0; s < n_splits; ++s) {
            float ls = l[(size_t)s * rows + r];
            if (!(ls > 0.0f)) continue;
            lt += ls * expf(m[(size_t)s * rows + r] - mx);
        }
        float inv = (isfinite(lt) && fabsf(lt) > MFO_L_EPS) ? 1.0f / lt : 0.0f;
        for (uint32_t d = 0; d < D; ++d) {
            float a = 0.0f;
            for (uint32_t s = 0; s < n_splits; ++s)
                a += acc[((size_t)s * rows + r) * D + d] * expf(m[(size_t)s * rows + r] - mx);
            out[(size_t)r * D + d] = mfo_f32_to_f16(a * inv);
        }
    }
}

/* ------------------------------------------------- 8-bit K/V cache (e4m3) ---
 * Not in the reference, which only has a roadmap for a quantised cache (docs/FLASH.md:121-186,
 * docs/SAGE.md:1-60).  Format defined by this project: K and V rows are stored as OCP FP8 E4M3
 * ("e4m3fn": 4 exponent bits, bias 7, 3 mantissa bits, largest finite 448, no infinity, NaN =
 * 0x7F) with one f32 scale per (page, kv head, row):
 *     amax  = max_i |x_i|            (x = the f16 row: K after RoPE and f16 rounding, V as given)
 *     scale = amax / 448  (1 when the row is all zeros)
 *     q_i   = e4m3_rne_satfinite(x_i / scale)           (IEEE f32 division)
 *     dequantised value = e4m3(q_i) * scale
 * Attention over such a cache follows the reference's contract with K := the decoded bytes
 * (products of the f16 q with the exactly-representable e4m3 values, f32 accumulation), the
 * row's scale applied to the score in f32, and V := dequantised rows. */

float mfo_e4m3_to_f32(uint8_t b)
{
    const uint32_t sign = b & 0x80u, exp = (b >> 3) & 0xFu, man = b & 7u;
    float v;
    if (exp == 0xFu && man == 7u) return NAN;
    if (exp == 0) v = ldexpf((float)man, -9);               /* subnormal: man * 2^-3 * 2^-6 */
    else v = ldexpf((float)(8u + man), (int)exp - 10);      /* (1 + man/8) * 2^(exp-7) */
    return sign ? -v : v;
}

/* f32 -> e4m3, round to nearest even, finite inputs saturate at +-448, NaN -> 0x7F
 * (the behaviour of cvt.rn.satfinite.e4m3x2.f32). */
uint8_t mfo_f32_to_e4m3(float x)
{
    if (isnan(x)) return 0x7F;
    const uint8_t sign = signbit(x) ? 0x80u : 0u;
    float a = fabsf(x);
    if (a >= 448.0f) return (uint8_t)(sign | 0x7E);
    if (a < ldexpf(1.0f, -10)) return sign; /* below half of the smallest subnormal (2^-9): 0 (ties to even -> 0) */
    int e;
    (void)frexpf(a, &e);                     /* a = f * 2^e, f in [0.5, 1) */
    int exp = e - 1;                         /* a = 1.xxx * 2^exp */
    if (exp < -6) exp = -6;                  /* subnormal range shares the exponent -6 */
    const float ulp = ldexpf(1.0f, exp - 3);
    float q = a / ulp;                       /* exact: power-of-two division */
    float r = rintf(q);                      /* current rounding mode: nearest even */
    float v = r * ulp;
    if (v >= 448.0f) return (uint8_t)(sign | 0x7E);
    /* encode v */
    if (v < ldexpf(1.0f, -6)) return (uint8_t)(sign | (uint8_t)(v / ldexpf(1.0f, -9)));
    (void)frexpf(v, &e);
    exp = e - 1;
    const uint32_t man = (uint32_t)(v / ldexpf(1.0f, exp - 3)) - 8u;
    return (uint8_t)(sign | ((uint32_t)(exp + 7) << 3) | man);
}

void mfo_quantize_row_e4m3(const uint16_t *x, uint32_t n, uint8_t *q, float *scale_out)
{
    h2f_init();
    float amax = 0.0f;
    for (uint32_t i = 0; i < n; ++i) {
        const float a = fabsf(H2F(x[i]));
        if (a > amax) amax = a;
    }
    const float scale = amax > 0.0f ? amax / 448.0f : 1.0f;
    for (uint32_t i = 0; i < n; ++i) q[i] = mfo_f32_to_e4m3(H2F(x[i]) / scale);
    *scale_out = scale;
}

/* Byte index of (cache row r, dim d) in the V pool of the 8-bit cache.  K rows lie row-major ([n_pages, Hkv, P, D]);
 * V is kept dim-major in blocks of 16 keys inside each (page, kv head) run of P rows - [n_pages, Hkv, P/16, D, 16] -
 * which is the operand layout of the 8-bit tensor-core product V^T W (page sizes are multiples of 16). */
size_t mfo_kv8_v_index(size_t r, uint32_t d, uint32_t head_dim, uint32_t page_size)
{
    const size_t in_page = r % page_size, run = r - in_page;
    return run * head_dim + (in_page / 16) * (16 * (size_t)head_dim) + (size_t)d * 16 + in_page % 16;
}

/* One new token per sequence appended to the 8-bit pools (K [n_pages, Hkv, P, D] bytes, V as mfo_kv8_v_index) with
 * scale pools [n_pages, Hkv, P] (f32): RoPE of q and k exactly as mfo_paged_kv_append, then the row quantiser. */
void mfo_paged_kv8_append(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint16_t *q_rot,
                          uint8_t *k_pool, uint8_t *v_pool, float *k_scales, float *v_scales,
                          const uint16_t *cos_t, const uint16_t *sin_t, const uint32_t *page_table,
                          uint32_t pt_stride, const uint32_t *positions, uint32_t batch, uint32_t n_heads,
                          uint32_t n_kv_heads, uint32_t head_dim, uint32_t page_size, uint32_t rope_mode,
                          int apply_rope)
{
    h2f_init();
    const uint32_t D = head_dim, half = D >> 1;
    uint16_t row[512];
    for (uint32_t b = 0; b < batch; ++b) {
        const uint32_t pos = positions[b];
        const uint16_t *c_row = cos_t + (size_t)pos * half, *s_row = sin_t + (size_t)pos * half;
        for (uint32_t h = 0; h < n_heads; ++h) {
            const uint16_t *src = q + ((size_t)b * n_heads + h) * D;
            for (uint32_t hd = 0; hd < D; ++hd)
                q_rot[((size_t)b * n_heads + h) * D + hd] = apply_rope ? rope_elem(src, c_row, s_row, hd, D, rope_mode) : src[hd];
        }
        const uint32_t page = page_table[(size_t)b * pt_stride + pos / page_size];
        for (uint32_t kh = 0; kh < n_kv_heads; ++kh) {
            const size_t r = ((size_t)page * n_kv_heads + kh) * page_size + pos % page_size;
            const uint16_t *ks = k + ((size_t)b * n_kv_heads + kh) * D, *vs = v + ((size_t)b * n_kv_heads + kh) * D;
            for (uint32_t hd = 0; hd < D; ++hd) row[hd] = apply_rope ? rope_elem(ks, c_row, s_row, hd, D, rope_mode) : ks[hd];
            mfo_quantize_row_e4m3(row, D, k_pool + r * D, k_scales + r);
            uint8_t vq[512];
            mfo_quantize_row_e4m3(vs, D, vq, v_scales + r);
            for (uint32_t hd = 0; hd < D; ++hd) v_pool[mfo_kv8_v_index(r, hd, D, page_size)] = vq[hd];
        }
    }
}

/* Decode attention of one sequence over an 8-bit paged cache: per-key online softmax in the order of
 * mfo_decode_online.  out is [Hq, D] f16 bits; gold (optional) the same in two-pass fp64 over the same
 * quantised data, [Hq, D] doubles. */
void mfo_decode_kv8(const uint16_t *q_rot, const uint8_t *k_pool, const uint8_t *v_pool, const float *k_scales,
                    const float *v_scales, const uint32_t *page_table_row, uint32_t kv_len, uint32_t n_heads,
                    uint32_t n_kv_heads, uint32_t head_dim, uint32_t page_size, float scale, uint16_t *out,
                    double *gold)
{
    h2f_init();
    const uint32_t D = head_dim, G = n_heads / n_kv_heads;
    double *sc = gold ? (double *)malloc(sizeof(double) * (kv_len ? kv_len : 1)) : NULL;
    for (uint32_t h = 0; h < n_heads; ++h) {
        const uint32_t kh = h / G;
        const uint16_t *qh = q_rot + (size_t)h * D;
        float m = MFO_NEG_SENTINEL, l = 0.0f, acc[512];
        for (uint32_t d = 0; d < D; ++d) acc[d] = 0.0f;
        double gmax = -1e300;
        for (uint32_t t = 0; t < kv_len; ++t) {
            const size_t r = ((size_t)page_table_row[t / page_size] * n_kv_heads + kh) * page_size + t % page_size;
            float dot = 0.0f;
            double gdot = 0.0;
            for (uint32_t d = 0; d < D; ++d) {
                const float kd = mfo_e4m3_to_f32(k_pool[r * D + d]);
                dot += H2F(qh[d]) * kd;
                gdot += (double)H2F(qh[d]) * (double)kd;
            }
            float score = (dot * k_scales[r]) * scale;
            if (!isfinite(score)) score = MFO_NEG_SENTINEL;
            if (gold) {
                sc[t] = gdot * (double)k_scales[r] * (double)scale;
                if (sc[t] > gmax) gmax = sc[t];
            }
            /* online step (streaming.metal:20-52) with the dequantised V row */
            const float mn = score > m ? score : m;
            const float alpha = expf(m - mn), w = expf(score - mn);
            l = l * alpha + w;
            for (uint32_t d = 0; d < D; ++d)
                acc[d] = acc[d] * alpha + w * (mfo_e4m3_to_f32(v_pool[mfo_kv8_v_index(r, d, D, page_size)]) * v_scales[r]);
            m = mn;
        }
        finish_decode_row(acc, l, D, out + (size_t)h * D);
        if (gold) {
            double lsum = 0.0;
            for (uint32_t d = 0; d < D; ++d) gold[(size_t)h * D + d] = 0.0;
            for (uint32_t t = 0; t < kv_len; ++t) {
                const size_t r = ((size_t)page_table_row[t / page_size] * n_kv_heads + kh) * page_size + t % page_size;
                const double w = exp(sc[t] - gmax);
                lsum += w;
                for (uint32_t d = 0; d < D; ++d)
                    gold[(size_t)h * D + d] += w * (double)mfo_e4m3_to_f32(v_pool[mfo_kv8_v_index(r, d, D, page_size)]) * (double)v_scales[r];
            }
            for (uint32_t d = 0; d < D; ++d) gold[(size_t)h * D + d] = lsum > 0.0 ? gold[(size_t)h * D + d] / lsum : 0.0;
        }
    }
    if (sc) free(sc);
}

/* ------------------------------------------------- materialised attention ---
 * SdpaReferenceStep / execute_sdpa_reference (src/metals/sdpa/step.rs:558-779) with the
 * rounding points of its three dispatches:
 *   1. S = scale * (Q K^T): f32 accumulation, alpha = scale applied to the sum, S stored
 *      as f16 scratch (step.rs:660-705; the scratch tensors are F16, sdpa/scratch.rs);
 *   2. row softmax of softmax_sdpa_batched.metal:14-115: masked entries (causal and
 *      i > row + query_offset) count as -INFINITY, max over the row, sum of exp(val - max)
 *      over the visible entries in f32, P = exp(val - max) / sum stored as f16; a row whose
 *      max or sum is not finite, or whose sum is <= 0, gets all-zero probabilities;
 *   3. O = P V: f16 x f16 products, f32 accumulation, stored as f16 (step.rs:735-776).
 * There is no GQA map: head h of Q uses head h of K and V (batch_stride_b per query head,
 * step.rs:690, 750), so the caches passed here are expanded [n_heads, k_rows, D].
 * Strides are in elements: q[h*q_stride_h + r*q_stride_m + d], out[h*out_stride_h +
 * r*out_stride_m + d].  expf stands in for metal::fast::exp. */
void mfo_sdpa_materialized(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint32_t n_heads,
                           uint32_t head_dim, uint32_t m, uint32_t kv_len, uint32_t k_rows,
                           uint32_t v_rows, uint64_t q_stride_h, uint64_t q_stride_m,
                           uint64_t out_stride_h, uint64_t out_stride_m, int causal,
                           uint32_t query_offset, float scale, uint16_t *out)
{
    h2f_init();
    const uint32_t D = head_dim;
    uint16_t *s16 = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)(kv_len ? kv_len : 1));
    uint16_t *p16 = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)(kv_len ? kv_len : 1));
    for (uint32_t h = 0; h < n_heads; ++h) {
        const uint16_t *kh = k + (size_t)h * k_rows * D;
        const uint16_t *vh = v + (size_t)h * v_rows * D;
        for (uint32_t r = 0; r < m; ++r) {
            const uint16_t *qr = q + (size_t)h * q_stride_h + (size_t)r * q_stride_m;
            const uint64_t mask_pos = (uint64_t)r + query_offset;
            for (uint32_t i = 0; i < kv_len; ++i) s16[i] = mfo_f32_to_f16(dot_f16(qr, kh + (size_t)i * D, D) * scale);
            float row_max = -INFINITY;
            for (uint32_t i = 0; i < kv_len; ++i) {
                float val = H2F(s16[i]);
                if (causal && i > mask_pos) val = -INFINITY;
                if (val > row_max) row_max = val;
            }
            float row_sum = 0.0f;
            if (isfinite(row_max))
                for (uint32_t i = 0; i < kv_len; ++i)
                    if (!causal || i <= mask_pos) row_sum += expf(H2F(s16[i]) - row_max);
            const int invalid = !isfinite(row_max) || !isfinite(row_sum) || row_sum <= 0.0f;
            for (uint32_t i = 0; i < kv_len; ++i) {
                float prob = 0.0f;
                if (!(causal && i > mask_pos) && !invalid) {
                    const float diff = H2F(s16[i]) - row_max;
                    prob = (isfinite(diff) ? expf(diff) : 0.0f) / row_sum;
                    if (!isfinite(prob)) prob = 0.0f;
                }
                p16[i] = mfo_f32_to_f16(prob);
            }
            uint16_t *dst = out + (size_t)h * out_stride_h + (size_t)r * out_stride_m;
            for (uint32_t d = 0; d < D; ++d) {
                float acc = 0.0f;
                for (uint32_t i = 0; i < kv_len; ++i) acc += H2F(p16[i]) * H2F(vh[(size_t)i * D + d]);
                dst[d] = mfo_f32_to_f16(acc);
            }
        }
    }
    free(s16);
    free(p16);
}

/* ------------------------------------------------------- timed CPU layer --- */

void mfo_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int mfo_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void mfo_paged_decode_layer(const uint16_t *q, const uint16_t *k, const uint16_t *v,
                            uint16_t *k_pool, uint16_t *v_pool, const uint16_t *cos_t,
                            const uint16_t *sin_t, const uint32_t *page_table, uint32_t pt_stride,
                            const uint32_t *kv_lens, uint32_t batch, uint32_t n_heads,
                            uint32_t n_kv_heads, uint32_t head_dim, uint32_t page_size,
                            uint32_t rope_mode, float scale, uint16_t *out)
{
    h2f_init();
    const uint32_t D = head_dim, half = D >> 1, G = n_heads / n_kv_heads;
#ifdef _OPENMP
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
#endif
    for (uint32_t b = 0; b < batch; ++b) {
        for (uint32_t kh = 0; kh < n_kv_heads; ++kh) {
            const uint32_t L = kv_lens[b];
            const uint32_t pos = L - 1;
            const uint32_t *pt = page_table + (size_t)b * pt_stride;
            const uint16_t *c_row = cos_t + (size_t)pos * half;
            const uint16_t *s_row = sin_t + (size_t)pos * half;
            /* append this kv head's row */
            {
                const uint16_t *ks = k + ((size_t)b * n_kv_heads + kh) * D;
                const uint16_t *vs = v + ((size_t)b * n_kv_heads + kh) * D;
                size_t slot = (((size_t)pt[pos / page_size] * n_kv_heads + kh) * page_size +
                               pos % page_size) * D;
                for (uint32_t hd = 0; hd < D; ++hd) {
                    k_pool[slot + hd] = rope_elem(ks, c_row, s_row, hd, D, rope_mode);
                    v_pool[slot + hd] = vs[hd];
                }
            }
            /* attend with the G query heads of this kv head */
            for (uint32_t g = 0; g < G; ++g) {
                uint32_t h = kh * G + g;
                uint16_t qr[256];
                float acc[256];
                const uint16_t *src = q + ((size_t)b * n_heads + h) * D;
                for (uint32_t hd = 0; hd < D; ++hd) qr[hd] = rope_elem(src, c_row, s_row, hd, D, rope_mode);
                float m = MFO_NEG_SENTINEL, l = 0.0f;
                for (uint32_t d = 0; d < D; ++d) acc[d] = 0.0f;
                for (uint32_t t = 0; t < L; ++t) {
                    size_t row = (((size_t)pt[t / page_size] * n_kv_heads + kh) * page_size +
                                  t % page_size) * D;
                    float score = dot_f16(qr, k_pool + row, D) * scale;
                    if (!isfinite(score)) score = MFO_NEG_SENTINEL;
                    online_step(score, v_pool + row, D, &m, &l, acc);
                }
                finish_decode_row(acc, l, D, out + ((size_t)b * n_heads + h) * D);
            }
        }
    }
}
