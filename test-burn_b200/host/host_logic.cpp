// Host-side logic of the KV-cache path that needs no device: RoPE table builder,
// capacity / growth rules, KV memory arithmetic and the prefill split-K selector.
// These mirror the reference's Rust host code so a caller sees the same numbers.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>
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


// KvGeometry::from_architecture (src/model/kv_geometry.rs:26-63).
mf_status mf_kv_geometry_from_architecture(uint32_t n_heads_in, uint32_t n_kv_heads_in, uint32_t d_model, MfKvGeometry *out)
{
    if (!out) return MF_ERR_INPUT_NOT_FOUND;
    const uint32_t n_heads = n_heads_in > 1 ? n_heads_in : 1;
    uint32_t n_kv = n_kv_heads_in == 0 ? n_heads : (n_kv_heads_in < n_heads ? n_kv_heads_in : n_heads);
    if (n_kv < 1) n_kv = 1;
    out->n_heads = n_heads;
    out->n_kv_heads = n_kv;
    out->group_size = (n_heads % n_kv == 0) ? n_heads / n_kv : 1;
    out->head_dim = d_model / n_heads;
    out->layout = n_kv < n_heads ? MF_KV_LAYOUT_COMPACT_KV_HEADS : MF_KV_LAYOUT_EXPANDED_HEADS;
    out->cache_heads = out->layout == MF_KV_LAYOUT_EXPANDED_HEADS ? n_heads : n_kv;
    return MF_OK;
}

// KvGeometry::from_cache_tensor (src/model/kv_geometry.rs:92-150), same checks in the same order,
// same messages.
mf_status mf_kv_geometry_from_cache_tensor(uint32_t n_heads, uint32_t n_kv_heads, uint32_t d_model, const MfTensor *t,
                                           uint64_t expected_capacity, MfKvGeometry *out, char *err, uint32_t err_len)
{
    if (err && err_len) err[0] = 0;
    if (!t || !out) return MF_ERR_INPUT_NOT_FOUND;
    MfKvGeometry base;
    mf_kv_geometry_from_architecture(n_heads, n_kv_heads, d_model, &base);
    auto bad = [&](const char *fmt, unsigned long long a, unsigned long long b, unsigned long long c) {
        if (err && err_len) snprintf(err, err_len, fmt, a, b, c);
        return MF_ERR_INVALID_SHAPE;
    };
    if (t->dtype != MF_DTYPE_F16) return bad("KV cache tensor must be F16, got dtype %llu", t->dtype, 0, 0);
    if (t->rank != 3) return bad("KV cache tensor must be rank-3 [heads, seq, head_dim], got rank %llu", t->rank, 0, 0);
    const uint64_t cache_heads = t->dims[0], seq = t->dims[1], head_dim = t->dims[2];
    if (seq != expected_capacity) return bad("KV cache capacity mismatch: got %llu, expected %llu", seq, expected_capacity, 0);
    if (head_dim != base.head_dim) return bad("KV cache head_dim mismatch: got %llu, expected %llu", head_dim, base.head_dim, 0);
    if (cache_heads == base.n_heads)
        base.layout = MF_KV_LAYOUT_EXPANDED_HEADS;
    else if (cache_heads == base.n_kv_heads)
        base.layout = MF_KV_LAYOUT_COMPACT_KV_HEADS;
    else
        return bad("KV cache heads mismatch: got %llu, expected %llu (expanded) or %llu (compact)", cache_heads, base.n_heads,
                   base.n_kv_heads);
    base.cache_heads = (uint32_t)cache_heads;
    *out = base;
    return MF_OK;
}

// ContextConfig::from_architecture (src/model/context.rs:105-152).
mf_status mf_context_config_from_architecture(uint64_t model_max, uint64_t override_len, uint64_t env_cap,
                                              uint32_t full_reserve, int64_t budget_mb, MfContextConfig *out)
{
    if (!out) return MF_ERR_INPUT_NOT_FOUND;
    const uint64_t cap = override_len ? override_len : env_cap;  // override_len.or(env_cap).filter(> 0)
    uint64_t max_len;
    if (model_max && cap)
        max_len = model_max < cap ? model_max : cap;
    else if (model_max)
        max_len = model_max;
    else if (cap)
        max_len = cap;
    else
        max_len = 2048;
    if (max_len < 1) max_len = 1;
    const uint64_t initial = full_reserve ? max_len : (max_len < 2048 ? max_len : 2048);
    out->max_context_len = max_len;
    out->allocated_capacity = mf_align_capacity(initial);
    out->full_reserve = full_reserve ? 1u : 0u;
    if (budget_mb >= 0) {
        out->budget_bytes = (uint64_t)budget_mb * 1024ull * 1024ull;
        out->budget_auto_pct = 0.f;
    } else {
        out->budget_bytes = 0;
        out->budget_auto_pct = 0.5f;
    }
    return MF_OK;
}

mf_status mf_context_config_from_env(uint64_t model_max, uint64_t override_len, MfContextConfig *out)
{
    auto parse = [](const char *name, bool trim, bool *ok) -> uint64_t {
        *ok = false;
        const char *v = getenv(name);
        if (!v) return 0;
        std::string sv(v);
        if (trim) {
            const size_t a = sv.find_first_not_of(" \t\r\n"), b = sv.find_last_not_of(" \t\r\n");
            sv = a == std::string::npos ? "" : sv.substr(a, b - a + 1);
        }
        if (sv.empty() || sv.find_first_not_of("0123456789") != std::string::npos) return 0;  // usize::parse
        *ok = true;
        return strtoull(sv.c_str(), nullptr, 10);
    };
    bool ok_cap = false, ok_mb = false;
    const uint64_t env_cap = parse("METALLIC_MAX_CONTEXT_LEN", true, &ok_cap);
    const uint64_t mb = parse("METALLIC_KV_MEMORY_BUDGET_MB", false, &ok_mb);
    return mf_context_config_from_architecture(model_max, override_len, ok_cap ? env_cap : 0,
                                               getenv("METALLIC_FULL_CONTEXT_RESERVE") != nullptr, ok_mb ? (int64_t)mb : -1, out);
}

// ContextConfig::apply_memory_budget (src/model/context.rs:158-210).
mf_status mf_apply_memory_budget(MfContextConfig *cfg, uint64_t device_recommended_bytes, uint64_t per_token_bytes)
{
    if (!cfg) return MF_ERR_INPUT_NOT_FOUND;
    uint64_t budget = cfg->budget_bytes;
    if (cfg->budget_auto_pct > 0.f) {
        const float pct = cfg->budget_auto_pct > 1.f ? 1.f : cfg->budget_auto_pct;
        budget = (uint64_t)((double)device_recommended_bytes * (double)pct);
    }
    if (per_token_bytes == 0 || budget == 0) return MF_OK;
    const uint64_t max_tokens = budget / per_token_bytes;
    if (max_tokens == 0) {
        cfg->max_context_len = 1;
        cfg->allocated_capacity = mf_align_capacity(1);
        return MF_OK;
    }
    const uint64_t budget_cap = mf_align_capacity(max_tokens);
    if (budget_cap < cfg->max_context_len) cfg->max_context_len = budget_cap;
    if (cfg->allocated_capacity > cfg->max_context_len) cfg->allocated_capacity = mf_align_capacity(cfg->max_context_len);
    return MF_OK;
}

}  // extern "C"
