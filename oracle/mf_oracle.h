/*
 * mf_oracle.h -- CPU restatement of the metallic-foundry KV-cache hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This library is the checker for the CUDA path:
 * it may be called from tests/, from the smoke entry and from the bench's
 * cpu-baseline leg, never from the product.  The product library does not link
 * it and has no CPU fallback.
 *
 * Provenance: the reference project is Rust + Metal and cannot be built or run
 * on a Linux/CUDA machine, so this is a scalar C restatement of its math, not
 * the reference's code running.  Each function names the reference file:line it
 * follows (paths are relative to crates/metallic-foundry/ of cchance27/test-burn).
 *
 * Pin status: the reference stores no expected outputs for this path (its tests
 * compare GPU against GPU, or GPU against a CPU function inside the test file).
 * What pins this oracle is therefore (1) the reference's deterministic test
 * input generator (an LCG) and test shapes, (2) identities the reference tests
 * assert (fused append == unfused chain bit-exact, identity RoPE, split == unsplit),
 * (3) an fp64 two-pass gold, and (4) an independent numpy restatement kept in
 * tests/.  For expected OUTPUT values of attention the parity is "unpinned":
 * there is no stored reference output anywhere to compare with.
 *
 * All tensors are IEEE binary16 stored as uint16_t unless noted.
 */
#ifndef MF_ORACLE_H
#define MF_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- binary16 <-> binary32, round-to-nearest-even, subnormals kept ---------
 * Stands in for half::f16::{from_f32,to_f32} (crate `half` 2.7.0 pinned in the
 * reference's Cargo.lock), which implements IEEE-754 RNE. */
uint16_t mfo_f32_to_f16(float x);
float mfo_f16_to_f32(uint16_t h);

/* ---- input generators ------------------------------------------------------ */

/* The reference's test LCG (tests/flashattention_decode_parity.rs:15-30):
 * state = state*1664525 + 1013904223; top 23 bits -> [0,1) -> (2u-1)*scale -> f16.
 * Returns the advanced state. */
uint32_t mfo_lcg_fill_f16(uint32_t state, uint16_t *out, size_t n, float scale);

/* Counter-based N(0,1) generator used for the benchmark-shaped inputs: element
 * i of stream (seed, tensor_id) is Box-Muller over two uniforms drawn from
 * splitmix64(seed ^ tensor_id*0x9E3779B97F4A7C15 ^ i).  Not from the reference. */
void mfo_normal_fill_f16(uint64_t seed, uint64_t tensor_id, uint64_t first,
                         uint16_t *out, size_t n);
uint64_t mfo_splitmix64(uint64_t x);

/* ---- RoPE tables (src/model/executor.rs:1980-2007) -------------------------
 * inv_freq_i = 1/powf(theta, 2i/D) [/ freq_factors[i]], angle = (float)p*inv_freq,
 * cosf/sinf in f32, one RNE to f16.  Rows [first_pos, first_pos+n_pos). */
void mfo_rope_tables(float theta, uint32_t head_dim, uint32_t first_pos,
                     uint32_t n_pos, const float *freq_factors,
                     uint16_t *cos_out, uint16_t *sin_out);

/* ---- unfused chain (the bit-exact definition of the cache contents) -------- */

/* tests/rope.rs:31-63 and src/metals/rope/rope.metal:36-74: NeoX half-split
 * RoPE over rows of `dim`; pos = (row % seq_len) + position_offset. */
void mfo_rope_neox(const uint16_t *in, uint16_t *out, const uint16_t *cos_t,
                   const uint16_t *sin_t, uint32_t dim, uint32_t seq_len,
                   uint32_t position_offset, size_t total_elements);

/* src/metals/kv_rearrange/kv_rearrange.metal:27-46: token-major [seq, row_stride]
 * -> head-major [n_heads, seq, head_dim]; source head = h / (n_heads/n_kv_heads). */
void mfo_kv_rearrange(const uint16_t *in, uint16_t *out, uint32_t row_stride,
                      uint32_t kv_head_dim, uint32_t n_heads, uint32_t n_kv_heads,
                      uint32_t head_dim, uint32_t seq);

/* tests/kv_cache.rs:14-32 / kv_cache_write.metal:17-29: [H, M, D] -> cache [H, cap, D]. */
void mfo_kv_cache_write(uint16_t *cache, const uint16_t *in, uint32_t n_kv_heads,
                        uint32_t head_dim, uint32_t input_seq_len,
                        uint32_t position_offset, uint32_t max_seq_len);

/* kv_cache_write_repeat.metal:24-39: same, each KV head replicated group_size
 * times into an expanded cache [n_kv_heads*group_size, cap, D]. */
void mfo_kv_cache_write_repeat(uint16_t *cache, const uint16_t *in, uint32_t n_kv_heads,
                               uint32_t group_size, uint32_t head_dim,
                               uint32_t input_seq_len, uint32_t position_offset,
                               uint32_t max_seq_len);

/* tests/kv_cache.rs:34-46 / kv_cache_read.metal:7-29: cache [H,cap,D] -> [H,L,D]. */
void mfo_kv_cache_read(const uint16_t *cache, uint16_t *out, uint32_t n_kv_heads,
                       uint32_t head_dim, uint32_t seq_len, uint32_t max_seq_len);

/* Growth copy (src/model/executor.rs:2493-2504): per head, current_pos rows move from the old
 * capacity's stride to the new one. */
void mfo_kv_cache_grow(const uint16_t *old_cache, uint16_t *new_cache, uint32_t heads, uint32_t head_dim,
                       uint32_t old_capacity, uint32_t new_capacity, uint32_t current_pos);

/* Contiguous cache rows [0, L) -> pages of one sequence (not in the reference). */
void mfo_paged_scatter(const uint16_t *cache, uint16_t *pool, const uint32_t *page_table_row, uint32_t L,
                       uint32_t n_kv_heads, uint32_t capacity, uint32_t page_size, uint32_t head_dim);

/* repeat_kv_heads.metal:11-44: [Hkv, L, D] -> [Hkv*G, L, D]. */
void mfo_repeat_kv_heads(const uint16_t *in, uint16_t *out, uint32_t n_kv_heads,
                         uint32_t group_size, uint32_t seq, uint32_t head_dim);

/* ---- fused QKV projection (src/metals/gemv/qkv_project.metal:4-272,
 *      src/metals/rmsnorm/rmsnorm.metal:18-95; CPU checks in tests/qkv_parity_f16.rs:18-69
 *      and tests/fused_qkv_batched_rmsnorm_parity.rs:23-56) ------------------------------
 * For each of the m rows of input [m, k_dim]:
 *   inv_rms = 1 / sqrt(sum(x^2) / k_dim + eps)            (f32, skipped when gamma == NULL)
 *   xn[k]   = f16((x[k] * inv_rms) * gamma[k])            (xn = x without gamma)
 *   out[r]  = f16(sum_k xn[k] * W[r, k] + bias[r])        (f32 sum in k order; bias may be NULL)
 * weights_per_block == 0: W row-major [N, k_dim]; otherwise the reference's blocked
 * ("canonical") layout: element (r, k) at (k % wpb) + wpb * (r + (k / wpb) * N). */
void mfo_fused_qkv(const uint16_t *input, const uint16_t *w_q, const uint16_t *w_k,
                   const uint16_t *w_v, const uint16_t *gamma, const uint16_t *b_q,
                   const uint16_t *b_k, const uint16_t *b_v, uint32_t m, uint32_t k_dim,
                   uint32_t n_dim, uint32_t n_kv, uint32_t weights_per_block, float eps,
                   uint16_t *out_q, uint16_t *out_k, uint16_t *out_v);

/* ---- fused append (src/metals/kv_prep/kv_prep_fused.metal:38-122) ---------- */
typedef struct {
    uint32_t d_model, kv_dim, head_dim, n_heads, n_kv_heads, group_size, seq_len,
        position_offset, max_seq_len, total_elements, rope_mode, layer_idx,
        no_rope_layer_step;
} mfo_kv_prep_params;

/* expanded != 0 writes each K/V row to the G heads of an [Hq, cap, D] cache. */
void mfo_kv_prep_fused(const uint16_t *q, const uint16_t *k, const uint16_t *v,
                       uint16_t *q_rot, uint16_t *k_cache, uint16_t *v_cache,
                       const uint16_t *cos_t, const uint16_t *sin_t,
                       const mfo_kv_prep_params *p, int expanded);

/* Paged append (layout defined by this project, not the reference): pools are
 * [n_pages, Hkv, P, D]; token t of sequence b lives at page_table[b*pt_stride + t/P],
 * row t%P.  One new token per sequence at position positions[b]; q is [B, Hq*D],
 * k,v are [B, Hkv*D]; q_rot is [B, Hq*D].  RoPE math as mfo_kv_prep_fused. */
void mfo_paged_kv_append(const uint16_t *q, const uint16_t *k, const uint16_t *v,
                         uint16_t *q_rot, uint16_t *k_pool, uint16_t *v_pool,
                         const uint16_t *cos_t, const uint16_t *sin_t,
                         const uint32_t *page_table, uint32_t pt_stride,
                         const uint32_t *positions, uint32_t batch, uint32_t n_heads,
                         uint32_t n_kv_heads, uint32_t head_dim, uint32_t page_size,
                         uint32_t rope_mode, int apply_rope);

/* Gather sequence b's first L tokens from a paged pool into [Hkv, L, D]. */
void mfo_paged_gather(const uint16_t *pool, const uint32_t *page_table_row,
                      uint32_t L, uint32_t n_kv_heads, uint32_t page_size,
                      uint32_t head_dim, uint16_t *out);

/* ---- decode attention ------------------------------------------------------
 * Q is [Hq, D] already roped and rounded to f16; caches are [cache_heads, cap, D];
 * kv head of query head h is h / (Hq / cache_heads) (flash_decode.metal:128-132).
 * Keys [key_begin, key_end) are visited.  Partial outputs are the unnormalised
 * f32 accumulator plus (m, l); pass acc/m/l == NULL to skip them. */

/* Per-key online softmax, the order of tests/sdpa_v2_parity.rs:85-130. */
void mfo_decode_online(const uint16_t *q_rot, const uint16_t *k_cache,
                       const uint16_t *v_cache, uint32_t n_heads, uint32_t cache_heads,
                       uint32_t head_dim, uint32_t capacity, uint32_t key_begin,
                       uint32_t key_end, float scale, uint16_t *out, float *acc,
                       float *m_out, float *l_out);

/* Block order of the reference kernel (flash_decode.metal:188-317): blocks of
 * `block_keys` keys, block max, weights exp(score - block_max), (m,l) update per
 * block, out = acc/l if |l|>1e-6 else acc, non-finite -> 0. */
void mfo_decode_blocked(const uint16_t *q_rot, const uint16_t *k_cache,
                        const uint16_t *v_cache, uint32_t n_heads, uint32_t cache_heads,
                        uint32_t head_dim, uint32_t capacity, uint32_t kv_len,
                        uint32_t block_keys, float scale, uint16_t *out);

/* Two-pass fp64 gold over the same f16 inputs; out_f64 is [Hq, D] doubles. */
void mfo_decode_gold(const uint16_t *q_rot, const uint16_t *k_cache,
                     const uint16_t *v_cache, uint32_t n_heads, uint32_t cache_heads,
                     uint32_t head_dim, uint32_t capacity, uint32_t kv_len, float scale,
                     double *out_f64);

/* The Rust CPU oracle of tests/sdpa_v2_parity.rs:37-133 as written there:
 * expanded K/V [B*H, L, D], NeoX RoPE of q at position L-1 and of every K row at
 * its own position, both rounded to f16, then the per-key online loop. */
void mfo_cpu_sdpa_attention(const uint16_t *q, const uint16_t *k, const uint16_t *v,
                            const uint16_t *cos_t, const uint16_t *sin_t,
                            uint32_t batch_heads, uint32_t kv_len, uint32_t head_dim,
                            uint16_t *out);

/* ---- causal prefill (flash_prefill.metal:158-269) --------------------------
 * Q [Hq, M, D] head-major (q_stride_h = M*D, q_stride_m = D), caches as above,
 * out token-major [M, Hq*D].  Key k visible to row r iff k <= r + query_offset.
 * 32-key tiles, block max, exp(score - block_max), per-tile (m,l,acc) update,
 * out = acc * (1/l) or 0.  tile_begin/tile_end (in 32-key tiles) restrict the
 * range for split-K; when acc != NULL the unnormalised partials are returned
 * ([Hq, M, D] f32, [Hq, M] m and l) and `out` may be NULL. */
void mfo_prefill_causal(const uint16_t *q, const uint16_t *k_cache, const uint16_t *v_cache,
                        uint32_t n_heads, uint32_t cache_heads, uint32_t head_dim,
                        uint32_t capacity, uint32_t q_len, uint32_t kv_len,
                        uint32_t query_offset, float scale, uint32_t tile_begin,
                        uint32_t tile_end, uint16_t *out, float *acc, float *m_out,
                        float *l_out);

void mfo_prefill_gold(const uint16_t *q, const uint16_t *k_cache, const uint16_t *v_cache,
                      uint32_t n_heads, uint32_t cache_heads, uint32_t head_dim,
                      uint32_t capacity, uint32_t q_len, uint32_t kv_len,
                      uint32_t query_offset, float scale, double *out_f64);

/* splitk_tile_range (flash_prefill.metal:452-457). */
void mfo_splitk_tile_range(uint32_t kv_len, uint32_t split_k, uint32_t split_id,
                           uint32_t *tile_begin, uint32_t *tile_end);

/* ---- split merge (flash_prefill.metal:843-888) -----------------------------
 * rows x n_splits partials: acc [n_splits, rows, D], m,l [n_splits, rows].
 * m* = max m_s; l* = sum over splits with l_s > 0 of l_s*exp(m_s - m*);
 * out = (sum acc_s*exp(m_s - m*)) / l*  (0 when l* is not finite or <= 1e-6). */
void mfo_merge_partials(const float *acc, const float *m, const float *l,
                        uint32_t n_splits, uint32_t rows, uint32_t head_dim,
                        uint16_t *out);

/* ---- 8-bit K/V cache (FP8 E4M3 with one f32 scale per cached row) --------------------
 * Not in the reference (roadmap only: docs/FLASH.md:121-186).  Format and arithmetic are
 * defined in mf_oracle.c above mfo_quantize_row_e4m3: scale = amax/448, q = rne_satfinite(x/scale),
 * value = e4m3(q) * scale; scores = (q . decoded bytes) * row scale * softmax scale in f32. */
float mfo_e4m3_to_f32(uint8_t b);
uint8_t mfo_f32_to_e4m3(float x);
void mfo_quantize_row_e4m3(const uint16_t *x, uint32_t n, uint8_t *q, float *scale_out);
/* byte index of (cache row r, dim d) in the V pool: dim-major blocks of 16 keys inside each (page, kv head) run */
size_t mfo_kv8_v_index(size_t r, uint32_t d, uint32_t head_dim, uint32_t page_size);
void mfo_paged_kv8_append(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint16_t *q_rot,
                          uint8_t *k_pool, uint8_t *v_pool, float *k_scales, float *v_scales,
                          const uint16_t *cos_t, const uint16_t *sin_t, const uint32_t *page_table,
                          uint32_t pt_stride, const uint32_t *positions, uint32_t batch, uint32_t n_heads,
                          uint32_t n_kv_heads, uint32_t head_dim, uint32_t page_size, uint32_t rope_mode,
                          int apply_rope);
void mfo_decode_kv8(const uint16_t *q_rot, const uint8_t *k_pool, const uint8_t *v_pool, const float *k_scales,
                    const float *v_scales, const uint32_t *page_table_row, uint32_t kv_len, uint32_t n_heads,
                    uint32_t n_kv_heads, uint32_t head_dim, uint32_t page_size, float scale, uint16_t *out,
                    double *gold);

/* ---- materialised attention (src/metals/sdpa/step.rs:558-779,
 *      src/metals/softmax/softmax_sdpa_batched.metal:14-115) --------------------
 * The reference's fallback path with its own rounding points: S = scale*QK^T stored as
 * f16, row softmax with a -INFINITY mask (causal: key i hidden from row r iff
 * i > r + query_offset), P stored as f16, O = P V.  No GQA map (head h of Q reads head h
 * of K/V): K is [n_heads, k_rows, D], V is [n_heads, v_rows, D].  Strides in elements.
 * This is the function the reference's flash-vs-materialised tests compare against. */
void mfo_sdpa_materialized(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint32_t n_heads,
                           uint32_t head_dim, uint32_t m, uint32_t kv_len, uint32_t k_rows,
                           uint32_t v_rows, uint64_t q_stride_h, uint64_t q_stride_m,
                           uint64_t out_stride_h, uint64_t out_stride_m, int causal,
                           uint32_t query_offset, float scale, uint16_t *out);

/* ---- timed CPU baseline ----------------------------------------------------
 * One layer of batched paged decode (append + attention) over `batch` sequences,
 * threaded with OpenMP over (sequence, kv head) when built with -fopenmp.
 * Same arithmetic as mfo_paged_kv_append + gather-free mfo_decode_online. */
void mfo_paged_decode_layer(const uint16_t *q, const uint16_t *k, const uint16_t *v,
                            uint16_t *k_pool, uint16_t *v_pool, const uint16_t *cos_t,
                            const uint16_t *sin_t, const uint32_t *page_table,
                            uint32_t pt_stride, const uint32_t *kv_lens, uint32_t batch,
                            uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                            uint32_t page_size, uint32_t rope_mode, float scale,
                            uint16_t *out);
int mfo_num_threads(void);
void mfo_set_num_threads(int n); /* launchers may export OMP_NUM_THREADS=1; the timed legs undo that */

#ifdef __cplusplus
}
#endif
#endif /* MF_ORACLE_H */
