// Host-side logic of the KV-cache path that needs no device: RoPE table builder,
// capacity / growth rules, KV memory arithmetic and the prefill split-K selector.
// These mirror the reference's Rust host code so a caller sees the same numbers.
#include <cmath>
#include <cstdint>
#include <vector>

#include <cuda_fp16.h>

#include "../../include/metallic_cuda.h"

namespace {

// IEEE binary32 -> binary16, round to nearest even (what half::f16::from_f32 does).
uint16_t f32_to_f16_rne(float x)
{
    return __half_as_ushort(__float2half_rn(x));
}

}  // namespace

extern "C" {

// src/model/executor.rs:1980-2007.  inv_freq and the angle are computed in f32,
// cos/sin by the f32 libm routines, then one rounding to f16.  `p as f32` is exact
// only up to 2^24 positions, as in the reference.
mf_status mf_rope_tables_host(float rope_base, uint32_t head_dim, uint32_t first_pos, uint32_t n_pos,
                              const float *freq_factors, uint16_t *cos_out, uint16_t *sin_out)
{
    if (!cos_out || !sin_out) return MF_ERR_INPUT_NOT_FOUND;
    if (head_dim == 0 || (head_dim & 1u)) return MF_ERR_INVALID_SHAPE;
    const uint32_t half = head_dim / 2;
    std::vector<float> inv(half);
    for (uint32_t i = 0; i < half; ++i) {
        const float exponent = (float)(2 * i) / (float)head_dim;
        float f = 1.0f / powf(rope_base, exponent);
        if (freq_factors) f /= freq_factors[i];
        inv[i] = f;
    }
    for (uint32_t r = 0; r < n_pos; ++r) {
        const float p = (float)(first_pos + r);
        for (uint32_t i = 0; i < half; ++i) {
            const float angle = p * inv[i];
            cos_out[(size_t)r * half + i] = f32_to_f16_rne(cosf(angle));
            sin_out[(size_t)r * half + i] = f32_to_f16_rne(sinf(angle));
        }
    }
    return MF_OK;
}

// ContextConfig::align_capacity (src/model/context.rs:213-219): multiples of 128, 0 -> 128.
uint64_t mf_align_capacity(uint64_t capacity)
{
    const uint64_t kAlign = 128;
    if (capacity == 0) return kAlign;
    return (capacity + kAlign - 1) / kAlign * kAlign;
}

// ensure_kv_capacity (src/model/executor.rs:2332-2396): a request that fits keeps the
// capacity; otherwise grow to max(2*current, required), clamp to the context limit,
// then align to 128 (the alignment is applied after the clamp, as in the reference).
// 0 = the request exceeds the context limit (the reference raises InvalidOperation).
uint64_t mf_grown_capacity(uint64_t current, uint64_t required, uint64_t max_context_len)
{
    if (required <= current) return current;
    if (required > max_context_len) return 0;
    uint64_t want = current * 2 > required ? current * 2 : required;
    if (want > max_context_len) want = max_context_len;
    return mf_align_capacity(want);
}

// KvGeometry::per_token_bytes_f16 (src/model/kv_geometry.rs:82-89).
uint64_t mf_kv_per_token_bytes_f16(uint32_t n_layers, uint32_t cache_heads, uint32_t head_dim)
{
    return (uint64_t)n_layers * 2ull * cache_heads * head_dim * 2ull;
}

// ContextConfig::estimate_kv_memory (src/model/context.rs:222-243).
uint64_t mf_estimate_kv_memory(uint32_t n_layers, uint32_t cache_heads, uint32_t head_dim, uint64_t context_len)
{
    const uint64_t per_layer = 2ull * cache_heads * context_len * head_dim * 2ull;
    return per_layer * n_layers;
}

// Split-K selector of the prefill dispatcher (src/metals/flashattention/step.rs:849-866).
uint32_t mf_prefill_split_k(uint32_t kv_seq_len, uint32_t q_seq_len)
{
    uint32_t split_k;
    if (kv_seq_len >= 4096 && q_seq_len >= 16)
        split_k = 8;
    else if (kv_seq_len >= 2048 && q_seq_len >= 16)
        split_k = 4;
    else
        split_k = 1;
    const uint32_t kv_tiles = (kv_seq_len + 31) / 32;
    const uint32_t cap = kv_tiles > 1 ? kv_tiles : 1;
    return split_k < cap ? split_k : cap;
}

}  // extern "C"
