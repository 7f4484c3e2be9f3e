/*
 * metallic_cuda.h -- C ABI of the B200 (sm_100a) KV-cache hot path for
 * metallic-foundry: fused RoPE + K/V append, flash-decode attention with
 * grouped-query heads (contiguous and paged caches, split-KV + log-sum-exp
 * merge) and causal chunked prefill.
 *
 * The reference project (cchance27/test-burn, crate metallic-foundry) has no C
 * ABI: its operators are Rust `Step`/`CompiledStep` impls that bind Metal
 * buffers.  Each entry point below names the reference item it replaces; paths
 * are relative to crates/metallic-foundry/.  The Rust side binds these symbols
 * with a plain `extern "C"` block.
 *
 * Conventions
 *  - All pointers inside MfTensor / the cache descriptors are DEVICE pointers
 *    valid on the context's device unless a parameter says "host".
 *  - The caller owns every buffer.  The library keeps no reference after a call
 *    returns, except for the context-owned scratch arena.
 *  - Every op is enqueued on the context's stream and returns without waiting.
 *  - A context is not thread-safe: one context per host thread per GPU.
 *  - Contract violations are rejected on the host before any launch (the Metal
 *    kernels silently return instead: flash_decode.metal:165-170).
 *  - There is no CPU fallback: if no CUDA device is present every call fails.
 */
#ifndef METALLIC_CUDA_H
#define METALLIC_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define MF_API __declspec(dllexport)
#else
#define MF_API __attribute__((visibility("default")))
#endif

/* ------------------------------------------------------------------ status ---
 * Mirrors the MetalError variants this path can raise (src/error.rs:22-75). */
typedef int32_t mf_status;
enum {
    MF_OK = 0,
    MF_ERR_OPERATION_NOT_SUPPORTED = 1, /* MetalError::OperationNotSupported */
    MF_ERR_INVALID_SHAPE = 2,           /* MetalError::InvalidShape */
    MF_ERR_INVALID_OPERATION = 3,       /* MetalError::InvalidOperation */
    MF_ERR_INPUT_NOT_FOUND = 4,         /* MetalError::InputNotFound (null tensor) */
    MF_ERR_UNSUPPORTED_DTYPE = 5,       /* MetalError::UnsupportedDtype */
    MF_ERR_OUT_OF_MEMORY = 6,           /* MetalError::OutOfMemory */
    MF_ERR_CUDA = 7,                    /* a CUDA runtime/driver call failed */
    MF_ERR_NCCL = 8,                    /* a collective failed */
    MF_ERR_TIMEOUT = 9                  /* a bounded device-side wait ran out */
};

/* ---------------------------------------------------------------- tensors ---
 * Replaces TensorArg (src/types/mod.rs:341-347): buffer + byte offset + dtype +
 * dims + element strides. */
enum { MF_DTYPE_F16 = 0, MF_DTYPE_F32 = 1, MF_DTYPE_U32 = 2 };

typedef struct MfTensor {
    void *dev_ptr;
    uint64_t offset_bytes;
    uint32_t dtype;
    uint32_t rank;
    uint64_t dims[4];
    uint64_t strides[4]; /* in elements */
} MfTensor;

/* ----------------------------------------------------------- param structs ---
 * Byte-for-byte the reference's #[repr(C)] structs (all fields 4 bytes). */

/* KvPrepFusedParamsResolved (src/metals/kv_prep/mod.rs:79-114). */
typedef struct KvPrepFusedParamsResolved {
    uint32_t d_model;
    uint32_t kv_dim;
    uint32_t head_dim;
    uint32_t n_heads;
    uint32_t n_kv_heads;
    uint32_t group_size;
    uint32_t seq_len;
    uint32_t position_offset;
    uint32_t max_seq_len;
    uint32_t total_elements;
    uint32_t rope_mode; /* 0 = neox (half-split), 1 = normal (adjacent pairs) */
    uint32_t layer_idx;
    uint32_t no_rope_layer_step;
} KvPrepFusedParamsResolved;
enum { MF_ROPE_MODE_NEOX = 0, MF_ROPE_MODE_NORMAL = 1 };

/* RopeParamsResolved (src/metals/rope/mod.rs:11-22). */
typedef struct RopeParamsResolved {
    uint32_t dim;
    uint32_t seq_len;
    uint32_t position_offset;
    uint32_t total_elements;
} RopeParamsResolved;

/* KvCacheWriteParamsResolved (src/metals/kv_cache_write/mod.rs:61-78). */
typedef struct KvCacheWriteParamsResolved {
    uint32_t n_kv_heads;
    uint32_t head_dim;
    uint32_t input_seq_len;
    uint32_t position_offset;
    uint32_t max_seq_len;
    uint32_t total_elements;
    uint32_t layer_idx;
} KvCacheWriteParamsResolved;

/* KvCacheWriteRepeatKvHeadsParamsResolved (src/metals/kv_cache_write/mod.rs:13-35). */
typedef struct KvCacheWriteRepeatKvHeadsParamsResolved {
    uint32_t n_kv_heads;
    uint32_t n_heads;
    uint32_t group_size;
    uint32_t head_dim;
    uint32_t input_seq_len;
    uint32_t position_offset;
    uint32_t max_seq_len;
    uint32_t total_elements;
    uint32_t layer_idx;
} KvCacheWriteRepeatKvHeadsParamsResolved;

/* SdpaParams (src/metals/flashattention/stages.rs:456-464). */
typedef struct SdpaParams {
    uint32_t kv_len;
    uint32_t head_dim;
    float scale;
    uint32_t stride_k_s;
    uint32_t stride_v_s;
} SdpaParams;

/* SdpaPrefillParams (src/metals/flashattention/stages.rs:240-270). */
typedef struct SdpaPrefillParams {
    uint32_t kv_len;
    uint32_t head_dim;
    float scale;
    uint32_t stride_k_s;
    uint32_t stride_v_s;
    uint32_t query_offset;
    uint32_t q_stride_b;
    uint32_t q_stride_h;
    uint32_t k_stride_b;
    uint32_t k_stride_h;
    uint32_t v_stride_b;
    uint32_t v_stride_h;
    uint32_t out_stride_b;
    uint32_t out_stride_h;
    uint32_t q_stride_m;
    uint32_t out_stride_m;
    uint32_t group_size;
    uint32_t q_len;
} SdpaPrefillParams;

/* SdpaPrefillSplitKParams (src/metals/flashattention/stages.rs:272-306). */
typedef struct SdpaPrefillSplitKParams {
    SdpaPrefillParams base;
    uint32_t n_heads;
    uint32_t split_k;
} SdpaPrefillSplitKParams;

/* Strides of one decode dispatch: FlashDecodeArgs minus the tensors
 * (src/metals/flashattention/step.rs:404-424). */
typedef struct MfFlashDecodeStrides {
    uint32_t q_stride_b, q_stride_h;
    uint32_t k_stride_b, k_stride_h;
    uint32_t v_stride_b, v_stride_h;
    uint32_t out_stride_b, out_stride_h;
} MfFlashDecodeStrides;

/* Fields of FlashAttentionStep after DynamicValue resolution
 * (src/metals/sdpa/step.rs:21-38). */
typedef struct MfFlashAttentionArgs {
    uint32_t causal;        /* bool */
    uint32_t query_offset;
    uint32_t n_heads;
    uint32_t head_dim;
    uint32_t kv_seq_len;
    uint32_t m;             /* 0 is treated as 1, like the reference */
    uint32_t kv_head_major; /* bool; must be 1 (sdpa/step.rs:193-197) */
} MfFlashAttentionArgs;

/* Which route the dispatcher took (for tests and logging). */
enum { MF_ROUTE_DECODE = 1, MF_ROUTE_PREFILL = 2, MF_ROUTE_PREFILL_SPLITK = 3, MF_ROUTE_REFERENCE = 4 };

/* ----------------------------------------------------------- paged KV cache ---
 * Not in the reference (its cache is contiguous only).  Pool layout per layer,
 * for K and for V: [n_pages, n_kv_heads, page_size, head_dim] f16.  Token t of
 * sequence b lives in page page_table[b*page_table_stride + t/page_size], row
 * t % page_size.  kv_lens[b] counts the tokens visible to the query AFTER the
 * append of this step (so the token appended by this step sits at kv_lens[b]-1). */
typedef struct MfPagedKv {
    void *k_pool;                /* device, f16 */
    void *v_pool;                /* device, f16 */
    const uint32_t *page_table;  /* device, [batch, page_table_stride] */
    const uint32_t *kv_lens;     /* device, [batch] */
    uint32_t n_pages;
    uint32_t n_kv_heads;
    uint32_t page_size;          /* 16, 32 or 64 */
    uint32_t head_dim;           /* 64 or 128 */
    uint32_t page_table_stride;
    uint32_t batch;
} MfPagedKv;

/* Inputs of one batched decode step over a paged cache: one new token per
 * sequence.  q is [batch, n_heads*head_dim], k and v are [batch, n_kv_heads*head_dim],
 * out is [batch, n_heads*head_dim]; cos/sin are [max_pos, head_dim/2] f16 tables. */
typedef struct MfPagedDecodeArgs {
    const void *q, *k, *v; /* device f16; k/v may be NULL when append == 0 */
    void *q_rot;           /* device f16 or NULL: optional copy of the roped q */
    void *out;             /* device f16 */
    const void *cos, *sin; /* device f16; may be NULL when rope == 0 */
    uint32_t n_heads;
    uint32_t rope;         /* 1: q (and appended k) are roped at position kv_lens[b]-1 */
    uint32_t rope_mode;    /* MF_ROPE_MODE_* */
    uint32_t append;       /* 1: write the new k,v row into the pool before attending */
    float scale;           /* 1/sqrt(head_dim), computed by the caller (step.rs:1042) */
} MfPagedDecodeArgs;

typedef struct MfContext MfContext;
typedef struct MfDecodePlan MfDecodePlan;

/* ------------------------------------------------------------------ context ---
 * Replaces Foundry (src/lib.rs:57-353): device + in-order stream + scratch. */
MF_API mf_status mf_context_create(int32_t device, void *cuda_stream, MfContext **out);
MF_API void mf_context_destroy(MfContext *ctx);
MF_API mf_status mf_context_set_stream(MfContext *ctx, void *cuda_stream);
MF_API mf_status mf_synchronize(MfContext *ctx); /* Foundry::synchronize (lib.rs:170-188) */
MF_API const char *mf_last_error(const MfContext *ctx);
MF_API const char *mf_status_name(mf_status s);
MF_API uint32_t mf_abi_version(void);
/* Number of kernels this context has launched since creation (instrumentation,
 * stands in for the per-dispatch metric events of lib.rs:225-233). */
MF_API uint64_t mf_launch_count(const MfContext *ctx);
/* Tuning knobs (the reference's are environment variables, docs/FLASH.md:204-225).
 * MF_OPTION_OVERLAP_LAUNCHES = 1: decode launches use programmatic dependent launch, so
 * the next launch's CTAs are scheduled while the previous grid drains.  A fused
 * append+decode launch then starts streaming K/V pages before the previous kernel in the
 * stream has finished; the caller promises that this previous kernel does not write the
 * pools, page table or lengths the launch reads (consecutive layers of a decode step never
 * do).  The library itself knows which of its own launches can still be in flight when a new
 * one starts (every eighth launch releases its dependents only after its own dependency wait,
 * which bounds that set by the launch protocol alone), keeps the caches those launches write
 * and does not stream early from one of them (a one-layer model, or two calls in a row on one
 * cache); kernels of other origins that release their dependents early are the caller's to
 * vouch for.  Everything else a launch reads or writes still waits for the previous kernel.
 * Value 2 extends the early streaming to launches WITHOUT a fused append (the shards of a
 * sequence-sharded step that do not own the tail page): the caller then also promises that no
 * separate append kernel precedes the launch in the stream.
 * MF_OPTION_DECODE_STAGES = n: depth of the decode kernel's K/V tile ring (0 = default).
 * MF_OPTION_PREFILL_IMPL: 0 = choose (tcgen05 kernel when the shape allows), 1 = mma.sync
 * kernel only, 2 = tcgen05 kernel only (like METALLIC_FA_PREFILL_* in the reference).
 * MF_OPTION_DECODE_CLUSTERS: 0 = short decode launches (few tiles per CTA, several CTAs per
 * (sequence, kv head) unit) run the CTAs of a unit as a thread-block cluster that combines
 * its states through distributed shared memory; 1 = never (every span writes a partial and
 * the last one merges, as long launches do).
 * MF_OPTION_QKV_IMPL: which kernel projects Q/K/V (mf_fused_qkv and its append forms): 0 = the
 * tcgen05 kernel from 8 input rows when the shape allows (k_dim a multiple of 128, n_dim and
 * n_kv of 128), else the mma.sync kernel; 1 = mma.sync kernel only; 2 = the tcgen05 kernel at
 * any row count the shape allows.
 * MF_OPTION_PLAN_ITEM_COST = n: what the step planner charges a CTA for every piece of a (sequence,
 * kv head) unit it takes, in 64-key tiles (0 = the default, 20): long launches give every CTA the
 * same tiles + n * pieces, not the same number of tiles.
 * MF_OPTION_PUSH_TAGGED: 1 (default) = mf_paged_decode_push_merge sends every float of a partial
 * together with the step's tag in one 8-byte store and the merging side trusts a word as soon as
 * it carries the tag, step + 1 (no system-scope fence, and nothing waits on the arrival counters,
 * which still advance so that steps of both forms may alternate; used when no rank is in
 * merge_only_mask); 0 = data, fence, arrival counters. */
enum {
    MF_OPTION_OVERLAP_LAUNCHES = 1,
    MF_OPTION_DECODE_STAGES = 2,
    MF_OPTION_PREFILL_IMPL = 3,
    MF_OPTION_DECODE_CLUSTERS = 4,
    MF_OPTION_QKV_IMPL = 5,
    MF_OPTION_PLAN_ITEM_COST = 6,
    MF_OPTION_PUSH_TAGGED = 7
};
MF_API mf_status mf_context_set_option(MfContext *ctx, uint32_t option, uint32_t value);
/* Caller-provided scratch (device); when absent the context allocates its own
 * arena on first use and grows it on demand (pooled scratch of step.rs:927-929). */
MF_API mf_status mf_context_set_scratch(MfContext *ctx, void *dev_ptr, uint64_t bytes);

/* ------------------------------------------------------- host-side builders ---
 * RoPE cos/sin tables (src/model/executor.rs:1980-2007), written to HOST f16
 * buffers of n_pos*head_dim/2 elements covering positions
 * [first_pos, first_pos+n_pos).  freq_factors may be NULL. */
MF_API mf_status mf_rope_tables_host(float rope_base, uint32_t head_dim, uint32_t first_pos,
                                     uint32_t n_pos, const float *freq_factors,
                                     uint16_t *cos_out, uint16_t *sin_out);

/* ContextConfig::align_capacity (src/model/context.rs:213-219). */
MF_API uint64_t mf_align_capacity(uint64_t capacity);
/* Growth rule of ensure_kv_capacity (src/model/executor.rs:2332-2396):
 * max(2*current, required) clamped to max_context_len, aligned to 128; returns 0
 * when required > max_context_len (the reference raises InvalidOperation). */
MF_API uint64_t mf_grown_capacity(uint64_t current, uint64_t required, uint64_t max_context_len);
/* KvGeometry::per_token_bytes_f16 (src/model/kv_geometry.rs:82-89). */
MF_API uint64_t mf_kv_per_token_bytes_f16(uint32_t n_layers, uint32_t cache_heads, uint32_t head_dim);
/* ContextConfig::estimate_kv_memory (src/model/context.rs:222-243), total bytes. */
MF_API uint64_t mf_estimate_kv_memory(uint32_t n_layers, uint32_t cache_heads, uint32_t head_dim,
                                      uint64_t context_len);
/* Prefill split-K heuristic (src/metals/flashattention/step.rs:849-866). */
MF_API uint32_t mf_prefill_split_k(uint32_t kv_seq_len, uint32_t q_seq_len);

/* KvCacheLayout / KvGeometry (src/model/kv_geometry.rs:6-90). */
enum { MF_KV_LAYOUT_EXPANDED_HEADS = 0, MF_KV_LAYOUT_COMPACT_KV_HEADS = 1 };
typedef struct MfKvGeometry {
    uint32_t n_heads;
    uint32_t n_kv_heads;
    uint32_t group_size;
    uint32_t head_dim;
    uint32_t layout;      /* MF_KV_LAYOUT_* */
    uint32_t cache_heads; /* n_heads (expanded) or n_kv_heads (compact) */
} MfKvGeometry;
/* KvGeometry::from_architecture (src/model/kv_geometry.rs:26-63) from the three architecture
 * numbers it reads: n_heads >= 1; n_kv_heads 0 means n_heads and is clamped to n_heads;
 * group_size = n_heads / n_kv_heads when that divides, else 1; head_dim = d_model / n_heads;
 * compact layout when n_kv_heads < n_heads, expanded otherwise.  (The reference can also
 * take the layout from the model file's cache tensor declaration; a caller that has one
 * overrides `layout` and `cache_heads` itself or uses mf_kv_geometry_from_cache_tensor.) */
MF_API mf_status mf_kv_geometry_from_architecture(uint32_t n_heads, uint32_t n_kv_heads, uint32_t d_model,
                                                  MfKvGeometry *out);
/* KvGeometry::from_cache_tensor (src/model/kv_geometry.rs:92-150): checks a cache tensor
 * against the architecture and returns the layout it implies.  MF_ERR_INVALID_SHAPE with the
 * reference's message in err (optional host buffer) when the tensor is not F16, not rank 3,
 * has another capacity than expected_capacity, another head_dim, or a head count that is
 * neither n_heads nor n_kv_heads. */
MF_API mf_status mf_kv_geometry_from_cache_tensor(uint32_t n_heads, uint32_t n_kv_heads, uint32_t d_model,
                                                  const MfTensor *cache, uint64_t expected_capacity,
                                                  MfKvGeometry *out, char *err, uint32_t err_len);

/* ContextConfig (src/model/context.rs:11-49). */
typedef struct MfContextConfig {
    uint64_t max_context_len;
    uint64_t allocated_capacity;
    uint64_t budget_bytes;      /* explicit budget; 0 with budget_auto_pct > 0 means "auto" */
    float budget_auto_pct;      /* MemoryBudget::Auto { percentage }; 0 when the budget is explicit */
    uint32_t full_reserve;      /* GrowthStrategy::FullReserve (else grow on demand from 2048, x2) */
} MfContextConfig;
/* ContextConfig::from_architecture (src/model/context.rs:105-152) as a pure function of what
 * it reads: the model's max_seq_len (0 = none), the caller's cap (0 = none), the value of
 * METALLIC_MAX_CONTEXT_LEN (0 = unset), whether METALLIC_FULL_CONTEXT_RESERVE is set, and
 * METALLIC_KV_MEMORY_BUDGET_MB (negative = unset -> Auto 50 %).  The caller's cap wins over
 * the environment's; either is clamped to the model's maximum; with neither a model maximum
 * nor a cap the limit is 2048; never below 1.  allocated_capacity = align(min(2048, max)),
 * or align(max) under full reserve. */
MF_API mf_status mf_context_config_from_architecture(uint64_t model_max_seq_len, uint64_t override_len,
                                                     uint64_t env_max_context_len, uint32_t full_reserve,
                                                     int64_t kv_memory_budget_mb, MfContextConfig *out);
/* The same, reading the three environment variables itself as the reference does. */
MF_API mf_status mf_context_config_from_env(uint64_t model_max_seq_len, uint64_t override_len, MfContextConfig *out);
/* ContextConfig::apply_memory_budget (src/model/context.rs:158-210): budget = the explicit
 * bytes, or pct x device_recommended_bytes; max tokens = budget / per_token_bytes; a budget
 * below one token pins both fields to 1 / align(1); otherwise max_context_len is lowered to
 * align(max tokens) when that is smaller, and allocated_capacity follows it down.
 * per_token_bytes comes from mf_kv_per_token_bytes_f16.  Nothing changes when either is 0. */
MF_API mf_status mf_apply_memory_budget(MfContextConfig *cfg, uint64_t device_recommended_bytes,
                                        uint64_t per_token_bytes);

/* ---------------------------------------------------------------- operators --- */

/* "KvPrepFused" (src/metals/kv_prep/step.rs:93-132, kv_prep_fused.metal:26-123):
 * q [M, Hq*D], k,v [M, Hkv*D] row-major -> q_rot [Hq, M, D] packed from element 0,
 * caches [cache_heads, max_seq_len, D] written at rows position_offset..+M.
 * The cache layout is taken from k_cache->dims[0]: Hkv = compact, Hq = expanded
 * (KvCacheLayout, src/model/kv_geometry.rs:6-12). */
MF_API mf_status mf_kv_prep_fused(MfContext *ctx, const MfTensor *q, const MfTensor *k,
                                  const MfTensor *v, const MfTensor *q_rot,
                                  const MfTensor *k_cache, const MfTensor *v_cache,
                                  const MfTensor *cos, const MfTensor *sin,
                                  const KvPrepFusedParamsResolved *params);

/* "Rope" (src/metals/rope/mod.rs, rope.metal:28-75): NeoX RoPE over rows of `dim`. */
MF_API mf_status mf_rope(MfContext *ctx, const MfTensor *input, const MfTensor *output,
                         const MfTensor *cos, const MfTensor *sin,
                         const RopeParamsResolved *params);

/* "KvCacheWrite" (kv_cache_write.metal:6-30): input [Hkv, M, D] -> rows
 * position_offset..+M of a compact cache [Hkv, cap, D]. */
MF_API mf_status mf_kv_cache_write(MfContext *ctx, const MfTensor *input, const MfTensor *cache,
                                   const KvCacheWriteParamsResolved *params);

/* "KvCacheWriteRepeatKvHeads" (kv_cache_write_repeat.metal:9-40): same input,
 * each KV head written to its group_size heads of an expanded cache [Hq, cap, D]. */
MF_API mf_status mf_kv_cache_write_repeat_kv_heads(MfContext *ctx, const MfTensor *input,
                                                   const MfTensor *cache,
                                                   const KvCacheWriteRepeatKvHeadsParamsResolved *params);

/* "KvRearrange" (src/metals/kv_rearrange/mod.rs:11-58, kv_rearrange.metal:10-47): projection rows
 * [batch*seq, row_stride] -> head-major [batch*n_heads, seq, head_dim], query head h reading kv
 * head h / (n_heads / n_kv_heads) at column kv_h * kv_head_dim + hd (skipped when >= kv_dim). */
typedef struct KvRearrangeParamsResolved {
    uint32_t kv_dim, row_stride, kv_head_dim, n_heads, n_kv_heads, head_dim, seq, total_elements;
} KvRearrangeParamsResolved;
MF_API mf_status mf_kv_rearrange(MfContext *ctx, const MfTensor *input, const MfTensor *output,
                                 const KvRearrangeParamsResolved *params);

/* "RepeatKvHeads" (src/metals/repeat_kv_heads/mod.rs:14-60, repeat_kv_heads.metal:11-44): cache
 * [batch*n_kv_heads, cache_stride, head_dim] -> [batch*n_heads, seq, head_dim], each kv head
 * repeated group_size times.  The attention routes of this library never need the repeated
 * copy (they index the compact cache); the op exists for callers of the unfused chain. */
typedef struct RepeatKvHeadsParamsResolved {
    uint32_t group_size, batch, n_kv_heads, n_heads, seq, head_dim, cache_stride, total_elements;
} RepeatKvHeadsParamsResolved;
MF_API mf_status mf_repeat_kv_heads(MfContext *ctx, const MfTensor *input, const MfTensor *output,
                                    const RepeatKvHeadsParamsResolved *params);

/* "KvCacheRead" (kv_cache_read.metal:7-29): cache [H, cap, D] -> [H, seq_len, D]. */
MF_API mf_status mf_kv_cache_read(MfContext *ctx, const MfTensor *cache, const MfTensor *output,
                                  uint32_t seq_len);

/* KV growth copy, preserve_kv_cache inside reallocate_kv_buffers
 * (src/model/executor.rs:2437-2513): rows [0, current_pos) of every head move from a
 * cache [heads, old_capacity, D] to one [heads, new_capacity, D]; the head stride changes
 * with the capacity, so the reference issues one blit per head - here one launch.  The
 * new capacity itself comes from mf_grown_capacity; RoPE tables are extended with
 * mf_rope_tables_host(first_pos = old length). */
MF_API mf_status mf_kv_cache_grow(MfContext *ctx, const MfTensor *old_cache, const MfTensor *new_cache,
                                  uint32_t current_pos);

/* "FlashAttention" (src/metals/sdpa/step.rs:160-503): the dispatcher.  m == 1 with
 * query_offset + 1 == kv_seq_len routes to decode, m > 1 (causal, query_offset + m ==
 * kv_seq_len) to prefill; anything else (non-causal, or an offset that breaks the causal
 * invariant) takes mf_sdpa_reference, as the reference falls back to its materialised
 * path there (MF_ROUTE_REFERENCE).  route_out may be NULL. */
/* "SdpaReference" (src/metals/sdpa/step.rs:89-158, execute_sdpa_reference :558-779,
 * softmax_sdpa_batched.metal:14-115): attention with the general mask, key i hidden from query
 * row r iff causal and i > r + query_offset; q and output layouts as in the prefill route.
 * The reference stores S and P as f16 scratch [Hq, m, kv_seq_len] and has no GQA map; here the
 * tiled kernels compute the same rows without scratch, with f32 softmax, and map query heads
 * to cache heads by the stride ratio like every other route. */
MF_API mf_status mf_sdpa_reference(MfContext *ctx, const MfTensor *q, const MfTensor *k, const MfTensor *v,
                                   const MfTensor *output, const MfFlashAttentionArgs *args);

MF_API mf_status mf_flash_attention(MfContext *ctx, const MfTensor *q, const MfTensor *k,
                                    const MfTensor *v, const MfTensor *output,
                                    const MfFlashAttentionArgs *args, uint32_t *route_out);

/* run_flash_decode (src/metals/flashattention/step.rs:558-585): decode when
 * q_seq_len == 1, prefill otherwise; strides inferred from the tensors exactly as
 * the reference does (q_rot head-major packed over the true M, cache capacity
 * from k->dims[1]). */
MF_API mf_status mf_run_flash_decode(MfContext *ctx, const MfTensor *q, const MfTensor *k,
                                     const MfTensor *v, const MfTensor *output, uint32_t n_heads,
                                     uint32_t head_dim, uint32_t kv_seq_len, uint32_t q_seq_len,
                                     uint32_t kv_head_major);

/* "FlashDecode" with explicit strides (src/metals/flashattention/step.rs:340-402;
 * kernels flash_decode.metal:146-490).  grid (1, n_heads, batch) in the reference;
 * here one CTA per (kv head, KV split, batch).  n_splits == 0 lets the library
 * choose. */
MF_API mf_status mf_flash_decode(MfContext *ctx, const void *q, const void *k, const void *v,
                                 void *output, const MfFlashDecodeStrides *strides,
                                 const SdpaParams *params, uint32_t n_heads, uint32_t batch,
                                 uint32_t n_splits);

/* Decode for callers that may not allocate device memory.  No counterpart in the
 * reference.  Same operation and arguments as mf_flash_decode (library-chosen split),
 * but it takes a bare stream instead of a context and calls no cudaMalloc, cudaFree
 * or other allocating routine: the split-KV partials and tickets live in a 4 MiB
 * array built into the library (resident on every GPU that loads the library, until
 * the process exits).  Meant for hosts whose own pool owns the whole GPU and forbids
 * plug-ins to allocate, for decode loops that cannot take the device-wide
 * synchronisation an allocation implies, and for sandboxes that deny the call.
 *  - Limit: batch x kv heads <= 4096 and (batch x kv heads + 2 x SM count) partial slots
 *    of 8*ceil(G/8)*(head_dim+2)*4 bytes within the 4 MiB; larger requests return
 *    MF_ERR_OUT_OF_MEMORY with a message and launch nothing.
 *  - The first call on a device looks the array's device address up and configures
 *    the kernels; make that first call before any stream capture begins.
 *  - All calls on a GPU share the array: calls that overlap on the GPU (other streams
 *    or threads) race; each call clears the status word and tickets on its stream.
 *  - err / err_len: optional host buffer for a message; a timed-out device-side wait
 *    is recorded in word 0 of the array, which this entry point does not read back:
 *    mf_static_scratch_status does, and the next call clears it.
 *  - Calls on one GPU must also be serialised by the host for the first-call set-up. */
MF_API mf_status mf_flash_decode_static_scratch(void *cuda_stream, const void *q, const void *k, const void *v,
                                                void *output, const MfFlashDecodeStrides *strides,
                                                const SdpaParams *params, uint32_t n_heads, uint32_t batch,
                                                char *err, uint32_t err_len);

/* Status word of the built-in array (no counterpart in the reference; allocates nothing):
 * enqueues one 4-byte copy on `cuda_stream` into *host_status (pinned memory keeps it
 * asynchronous).  Once the stream has drained, non-zero means that a device-side wait of
 * the last mf_flash_decode_static_scratch call on the current GPU ran out and that its
 * output must not be used. */
MF_API mf_status mf_static_scratch_status(void *cuda_stream, uint32_t *host_status);

/* RopeFlashDecodeStep (src/metals/flashattention/step.rs:54-306): NeoX RoPE of q
 * at rope->position_offset fused in front of decode.  q is un-roped [batch, Hq, D]. */
MF_API mf_status mf_rope_flash_decode(MfContext *ctx, const void *q, const void *k, const void *v,
                                      const void *cos, const void *sin, void *output,
                                      const RopeParamsResolved *rope, const SdpaParams *params,
                                      const MfFlashDecodeStrides *strides, uint32_t n_heads,
                                      uint32_t batch);

/* Causal prefill with explicit params (flash_prefill.metal:94-446 and the
 * split-K pair :460-983).  split_k <= 1 runs the single kernel. */
MF_API mf_status mf_flash_prefill(MfContext *ctx, const void *q, const void *k, const void *v,
                                  void *output, const SdpaPrefillSplitKParams *params);

/* Split merge (flash_prefill.metal:806-983), also the merge that follows the
 * cross-GPU all-gather: acc [n_splits, rows, D] f32, m,l [n_splits, rows] f32
 * -> out [rows, D] f16. */
MF_API mf_status mf_merge_partials(MfContext *ctx, const float *acc, const float *m,
                                   const float *l, uint32_t n_splits, uint32_t rows,
                                   uint32_t head_dim, void *out);

/* The same merge over an all-gathered buffer: split s of acc / m / l starts
 * split_stride floats after split s-1 (e.g. each rank sends [acc | m | l] as one block of
 * rows*(head_dim+2) floats and split_stride is that block size). */
MF_API mf_status mf_merge_partials_strided(MfContext *ctx, const float *acc, const float *m,
                                           const float *l, uint32_t n_splits, uint32_t rows,
                                           uint32_t head_dim, uint64_t split_stride, void *out);

/* ------------------------------------------------------ paged batched decode ---
 * No counterpart in the reference (contiguous cache, batch 1).  A plan cuts the
 * step's KV tiles into spans of equal cost (tiles + a charge per piece of a
 * (sequence, kv head) unit), one per resident CTA; it depends only on
 * kv_lens (host copy), geometry and the device, and is reused by every layer of
 * the step. */
MF_API mf_status mf_decode_plan_create(MfContext *ctx, const uint32_t *kv_lens_host, uint32_t batch,
                                       uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                                       uint32_t page_size, uint32_t max_ctas, MfDecodePlan **out);
/* Re-plan in place for new lengths (same batch and geometry); no allocation when
 * the work list fits the plan's capacity. */
MF_API mf_status mf_decode_plan_update(MfContext *ctx, MfDecodePlan *plan,
                                       const uint32_t *kv_lens_host);
MF_API void mf_decode_plan_destroy(MfContext *ctx, MfDecodePlan *plan);
/* The planner alone, on the host (no device needed): fills items_out (8 uint32 per
 * item: seq, kvh, tile_begin, tile_end, slot, unit, n_parts, first_slot) and
 * cta_begin_out (n_ctas+1 entries); returns the number of items, or the number
 * needed when item_capacity is too small.  n_ctas_out receives the CTA count. */
MF_API uint32_t mf_decode_plan_build_host(const uint32_t *kv_lens_host, uint32_t batch, uint32_t n_kv_heads,
                                          uint32_t max_ctas, uint32_t *items_out, uint32_t item_capacity,
                                          uint32_t *cta_begin_out, uint32_t *n_ctas_out);
/* The same for launches the library may run in the cluster form (at most one CTA per SM): max_cluster is the
 * largest cluster size allowed (a power of two up to 16, 0 = none), clusters_of_16 / clusters_of_8 how many
 * clusters of those sizes the device holds at once (0 = no limit).  *cluster_out: the cluster size chosen, 0 =
 * plain form (then the result is mf_decode_plan_build_host's); in the cluster form every item is one range of
 * one unit and one cluster, *n_ranges_out their number (CTAs = ranges * cluster size). */
MF_API uint32_t mf_decode_plan_build_host_clusters(const uint32_t *kv_lens_host, uint32_t batch, uint32_t n_kv_heads,
                                                   uint32_t max_ctas, uint32_t max_cluster, uint32_t clusters_of_16,
                                                   uint32_t clusters_of_8, uint32_t *items_out, uint32_t item_capacity,
                                                   uint32_t *n_ranges_out, uint32_t *cluster_out);
MF_API uint32_t mf_decode_plan_ctas(const MfDecodePlan *plan);
/* CTAs per thread-block cluster of the plan's launches (0: the plain form, see MF_OPTION_DECODE_CLUSTERS). */
MF_API uint32_t mf_decode_plan_cluster(const MfDecodePlan *plan);
MF_API uint32_t mf_decode_plan_items(const MfDecodePlan *plan);
MF_API uint64_t mf_decode_plan_tiles(const MfDecodePlan *plan);

/* Append (optional) + RoPE (optional) + GQA flash-decode over a paged cache, one
 * launch per layer. */
MF_API mf_status mf_paged_decode(MfContext *ctx, const MfDecodePlan *plan, const MfPagedKv *cache,
                                 const MfPagedDecodeArgs *args);

/* Stand-alone paged append (RoPE + K/V slot write, q_rot out) for M new tokens of
 * sequence `seq` starting at position_offset (chunked prefill into a paged cache),
 * or with seq == UINT32_MAX one token per sequence at kv_lens[b]-1. */
MF_API mf_status mf_paged_kv_append(MfContext *ctx, const MfPagedKv *cache, const void *q,
                                    const void *k, const void *v, void *q_rot, const void *cos,
                                    const void *sin, uint32_t n_heads, uint32_t rope_mode,
                                    uint32_t apply_rope, uint32_t seq, uint32_t position_offset,
                                    uint32_t seq_len);

/* KvPrepFused and the decode route of FlashAttention in ONE launch, for one new token (seq_len = 1) on a
 * compact contiguous cache: q is rotated on its way into the kernel (and stored to q_rot when q_rot is
 * not NULL), the new key is rotated, the new K/V rows are written to cache row position_offset, and
 * attention runs over rows [0, position_offset] -- the same bits in the caches and in q_rot as
 * mf_kv_prep_fused, the same attention as mf_flash_attention after it.  An expanded cache
 * ([n_heads, cap, D]) is answered with MF_ERR_OPERATION_NOT_SUPPORTED: use the two calls.  No
 * counterpart in the reference, which launches the two steps one after the other
 * (src/metals/kv_prep/step.rs:93-132, src/metals/sdpa/step.rs:160-503). */
MF_API mf_status mf_kv_prep_flash_decode(MfContext *ctx, const MfTensor *q, const MfTensor *k, const MfTensor *v,
                                         const MfTensor *q_rot, const MfTensor *k_cache,
                                         const MfTensor *v_cache, const MfTensor *cos, const MfTensor *sin,
                                         const MfTensor *output, const KvPrepFusedParamsResolved *params);

/* ------------------------------------------- projection in front of the append --- */

/* "FusedQkv" (src/metals/gemv/qkv_step.rs:14-37,59-101; qkv_project.metal:4-272), f16 weights
 * (the reference's F16 policy; its block-quantised policies are not built):
 *   inv_rms = 1 / sqrt(mean(x^2) + epsilon), xn = f16((x * inv_rms) * gamma)   (gamma NULL: xn = x)
 *   out_q[r] = f16(sum_k xn[k] * Wq[r, k] + bias_q[r]), same for K and V        (bias NULL: none)
 * input [m, k_dim], out_q [m, n_dim], out_k / out_v [m, n_kv], all f16 row-major.
 * weights_per_block == 0: weights row-major [N, k_dim]; 32: the reference's blocked layout, element
 * (r, k) at (k % 32) + 32 * (r + (k / 32) * N) (compound/stages/layout.rs:100).  k_dim must be a
 * multiple of 32, n_dim and n_kv multiples of 16.  Sums are f32 in a fixed order that does not depend
 * on m or on which entry point runs, so the three functions below produce the same bits.
 * The weights, gamma excepted, are treated as constants of the stream: with MF_OPTION_OVERLAP_LAUNCHES
 * set the kernel is a programmatic dependent of the launch before it and requests its first weights
 * before that launch has finished, so the preceding kernel in the stream must not be the one that
 * writes them.  Input rows, gamma and biases are read, and everything is written, after the wait.
 * Up to eight input rows share one pass over the weights; more rows repeat the pass per eight. */
typedef struct MfFusedQkvArgs {
    const void *input;
    const void *w_q, *w_k, *w_v;
    const void *gamma;                      /* f16 [k_dim] or NULL */
    const void *bias_q, *bias_k, *bias_v;   /* f16, all three or none */
    void *out_q, *out_k, *out_v;            /* may be NULL in the two append forms */
    uint32_t k_dim, n_dim, n_kv, m;
    uint32_t weights_per_block;
    float epsilon;
} MfFusedQkvArgs;
MF_API mf_status mf_fused_qkv(MfContext *ctx, const MfFusedQkvArgs *args);

/* FusedQkv followed by KvPrepFused in ONE launch: the projected rows never reach memory as q/k/v
 * (unless out_* are given); each is rounded to f16 exactly as the two-launch sequence would store
 * it, rotated, and written to q_rot / the caches.  Same bits as mf_fused_qkv then mf_kv_prep_fused.
 * args->m = params->seq_len, n_dim = n_heads*head_dim, n_kv = n_kv_heads*head_dim.  No counterpart
 * in the reference, which runs the two steps back to back (models/qwen25.json layer block). */
MF_API mf_status mf_fused_qkv_kv_prep(MfContext *ctx, const MfFusedQkvArgs *args, const MfTensor *q_rot,
                                      const MfTensor *k_cache, const MfTensor *v_cache,
                                      const MfTensor *cos, const MfTensor *sin,
                                      const KvPrepFusedParamsResolved *params);

/* The same in front of a paged cache: arguments after `args` as mf_paged_kv_append (seq_len = args->m). */
MF_API mf_status mf_fused_qkv_paged_append(MfContext *ctx, const MfFusedQkvArgs *args,
                                           const MfPagedKv *cache, void *q_rot, const void *cos,
                                           const void *sin, uint32_t n_heads, uint32_t rope_mode,
                                           uint32_t apply_rope, uint32_t seq, uint32_t position_offset);

/* Migration of a contiguous compact cache [Hkv, capacity, D] into the pages of sequence
 * `seq`: rows [0, len) of every kv head (K pool when use_v == 0, V pool otherwise).  No
 * counterpart in the reference; the inverse of mf_paged_gather. */
MF_API mf_status mf_kv_cache_to_pages(MfContext *ctx, const MfTensor *cache, const MfPagedKv *paged,
                                      uint32_t use_v, uint32_t seq, uint32_t len);

/* Causal chunked prefill attention over the PAGES of sequence `seq` (after mf_paged_kv_append has put
 * the chunk's rows there): the math of mf_flash_prefill (flash_prefill.metal:94-446, split-K
 * :452-983), K/V tiles fetched page by page through the page table.  Key k is visible to query row
 * r iff k <= r + query_offset; q rows are at q + head * q_stride_h + r * q_stride_m (elements), out
 * likewise; kv_len keys of the sequence are attended.  No counterpart in the reference. */
typedef struct MfPagedPrefillArgs {
    const void *q;
    void *out;
    uint32_t seq, q_len, kv_len, query_offset, n_heads;
    uint32_t q_stride_h, q_stride_m, out_stride_h, out_stride_m;
    float scale;
} MfPagedPrefillArgs;
MF_API mf_status mf_paged_prefill(MfContext *ctx, const MfPagedKv *cache, const MfPagedPrefillArgs *args);

/* Debug/oracle gather: first `len` tokens of sequence `seq` -> [Hkv, len, D]. */
MF_API mf_status mf_paged_gather(MfContext *ctx, const MfPagedKv *cache, uint32_t use_v,
                                 uint32_t seq, uint32_t len, void *out);

/* Sequence-sharded decode: this shard attends over its own keys only and emits
 * unnormalised f32 partials (acc [batch, Hq, D], m and l [batch, Hq]) for the
 * all-gather + mf_merge_partials step.  kv_lens in `cache` are the shard-local
 * lengths; positions for RoPE come from rope_positions (device, [batch]). */
MF_API mf_status mf_paged_decode_partial(MfContext *ctx, const MfDecodePlan *plan,
                                         const MfPagedKv *cache, const MfPagedDecodeArgs *args,
                                         const uint32_t *rope_positions, float *acc, float *m,
                                         float *l);

/* ---- paged cache life cycle: page allocator and prefix cache (host) ---------------------
 * Replaces the reference's prefix snapshots (src/model/executor.rs:1136-1675): same
 * entry rules (at most max_entries, default 8, clamped to 1..64; a store replaces the entry of
 * the same key, or without key of the same tokens, and drops the oldest when full; a lookup
 * without key takes the longest snapshot that is a prefix of the prompt, with key the longest
 * common prefix among that key's entries not longer than the prompt; later entry on ties; a hit
 * moves the entry to the back), but a snapshot is a list of page ids with raised reference
 * counts instead of a copy of the rows.  Not thread-safe: one owner, like a context. */
typedef struct MfPagePool MfPagePool;
typedef struct MfPrefixCache MfPrefixCache;
MF_API mf_status mf_page_pool_create(uint32_t n_pages, MfPagePool **out);
MF_API void mf_page_pool_destroy(MfPagePool *pool);
/* n pages with reference count 1, or MF_ERR_OUT_OF_MEMORY and none. */
MF_API mf_status mf_page_pool_alloc(MfPagePool *pool, uint32_t n, uint32_t *ids_out);
MF_API mf_status mf_page_pool_retain(MfPagePool *pool, const uint32_t *ids, uint32_t n);
/* A page returns to the free list when its count reaches zero. */
MF_API mf_status mf_page_pool_release(MfPagePool *pool, const uint32_t *ids, uint32_t n);
MF_API uint32_t mf_page_pool_free_count(const MfPagePool *pool);
MF_API uint32_t mf_page_pool_refcount(const MfPagePool *pool, uint32_t id);
MF_API uint32_t mf_prefix_cache_default_entries(void);
MF_API mf_status mf_prefix_cache_create(MfPagePool *pool, uint32_t page_size, uint32_t max_entries,
                                        MfPrefixCache **out);
/* Releases the pages its entries hold. */
MF_API void mf_prefix_cache_destroy(MfPrefixCache *cache);
MF_API uint32_t mf_prefix_cache_entries(const MfPrefixCache *cache);
/* page_ids: the ceil(n_tokens / page_size) pages holding the prefix; they are retained. */
MF_API mf_status mf_prefix_cache_store(MfPrefixCache *cache, const uint32_t *tokens, uint32_t n_tokens,
                                       const char *key, const uint32_t *page_ids, uint32_t n_pages);
/* On a hit *matched_out tokens are covered by the first *n_pages_out ids written to
 * page_ids_out, each retained for the caller.  When matched % page_size != 0, or the caller
 * will append into the last page, that page must be replaced by a private copy first
 * (mf_page_pool_alloc + mf_paged_copy_pages + release of the shared id). */
MF_API mf_status mf_prefix_cache_lookup(MfPrefixCache *cache, const uint32_t *prompt, uint32_t n_prompt,
                                        const char *key, uint32_t *matched_out, uint32_t *page_ids_out,
                                        uint32_t page_ids_cap, uint32_t *n_pages_out);
/* Copies whole pages (all kv heads, K and V pools) dst_ids[i] <- src_ids[i]; ids are device arrays. */
MF_API mf_status mf_paged_copy_pages(MfContext *ctx, const MfPagedKv *cache, const uint32_t *src_ids,
                                     const uint32_t *dst_ids, uint32_t n);

/* ---- 8-bit K/V cache (FP8 E4M3, one f32 scale per cached row) ------------------------
 * The reference has only a roadmap for a quantised cache (docs/FLASH.md:121-186,
 * docs/SAGE.md:1-60); the format here is this project's.  Byte pools of n_pages * n_kv_heads *
 * page_size * 128 bytes for K and for V, every byte an OCP FP8 E4M3 value, and scale pools
 * [n_pages, n_kv_heads, page_size] f32: for a row x (K after RoPE and f16 rounding, V as
 * given) amax = max |x_i|, scale = amax / 448 (1 for an all-zero row), byte_i =
 * e4m3 round-to-nearest-even, saturating, of x_i / scale; the cached value is byte * scale.
 * K is row-major, [n_pages, n_kv_heads, page_size, 128].  V is dim-major in blocks of 16 keys
 * inside each (page, kv head) run, [n_pages, n_kv_heads, page_size / 16, 128, 16]: byte (row r
 * of the page, dim d) at (r / 16) * 2048 + d * 16 + r % 16 - the operand layout of V^T W on the
 * tensor cores, so that V's bytes need no transposition on their way into the product.
 * head_dim 128 only, page_size 16, 32 or 64, GQA groups of up to 8 heads.
 * Attention over it keeps the reference's contract with K := decoded bytes * row scale and
 * V := dequantised rows; half the bytes of the f16 cache cross HBM per key. */
typedef struct MfPagedKv8 {
    void *k_pool;                /* device, bytes */
    void *v_pool;
    float *k_scales;             /* device, f32 */
    float *v_scales;
    const uint32_t *page_table;  /* device, [batch, page_table_stride] */
    const uint32_t *kv_lens;     /* device, [batch] */
    uint32_t n_pages;
    uint32_t n_kv_heads;
    uint32_t page_size;
    uint32_t head_dim;           /* 128 */
    uint32_t page_table_stride;
    uint32_t batch;
} MfPagedKv8;
/* mf_paged_decode over the 8-bit cache: optional append (RoPE of k, row quantiser, pool and scale
 * written) + RoPE of q + GQA flash-decode in one launch.  Plans in the plain and in the cluster form are
 * taken (where the device refuses the plan's cluster size every range runs as one CTA's item). */
MF_API mf_status mf_paged_decode_kv8(MfContext *ctx, const MfDecodePlan *plan, const MfPagedKv8 *cache,
                                     const MfPagedDecodeArgs *args);
/* Causal chunked prefill over the 8-bit cache (mf_paged_prefill's arguments): the sequence's first kv_len rows are
 * dequantised (e4m3 * row scale, rounded to f16) into the caller's workspace as K and V [Hkv, kv_len, D], then the
 * f16 prefill kernels run on them.  workspace: device memory, 256-byte aligned, at least
 * mf_paged_prefill_kv8_workspace_bytes(cache, kv_len) bytes; the library allocates nothing. */
MF_API uint64_t mf_paged_prefill_kv8_workspace_bytes(const MfPagedKv8 *cache, uint32_t kv_len);
MF_API mf_status mf_paged_prefill_kv8(MfContext *ctx, const MfPagedKv8 *cache, const MfPagedPrefillArgs *args,
                                      void *workspace, uint64_t workspace_bytes);
/* mf_paged_decode_partial over the 8-bit cache: this shard attends over its own keys only and emits
 * unnormalised f32 partials (acc [batch, Hq, D] 16-byte aligned, m and l [batch, Hq]) for mf_merge_partials,
 * mf_allgather_merge or any other gather; kv_lens in `cache` are the shard-local lengths, RoPE positions come
 * from rope_positions (device, [batch]; may be null when args->rope and args->append are 0); args->out is not
 * written.  No counterpart in the reference. */
MF_API mf_status mf_paged_decode_kv8_partial(MfContext *ctx, const MfDecodePlan *plan, const MfPagedKv8 *cache,
                                             const MfPagedDecodeArgs *args, const uint32_t *rope_positions, float *acc,
                                             float *m, float *l);
/* mf_paged_kv_append for the 8-bit cache (same arguments and q_rot layouts): seq == 0xFFFFFFFF
 * appends one token per sequence at kv_lens[b] - 1, otherwise seq_len rows of sequence `seq`
 * at position_offset (a prefill chunk). */
MF_API mf_status mf_paged_kv8_append(MfContext *ctx, const MfPagedKv8 *cache, const void *q, const void *k,
                                     const void *v, void *q_rot, const void *cos, const void *sin, uint32_t n_heads,
                                     uint32_t rope_mode, uint32_t apply_rope, uint32_t seq, uint32_t position_offset,
                                     uint32_t seq_len);
/* The first `len` rows of one sequence, dequantised, as a contiguous [n_kv_heads, len, 128] f16 cache. */
MF_API mf_status mf_paged_kv8_gather(MfContext *ctx, const MfPagedKv8 *cache, uint32_t use_v, uint32_t seq,
                                     uint32_t len, void *out);

/* ---- sequence-sharded decode with the exchange fused into the kernels ---------------
 * No counterpart in the reference.  Instead of all-gathering (acc, m, l) with a
 * library collective, the decode kernel of every rank stores each finished unit's
 * partial directly into every rank's receive block (plain peer stores over NVLink),
 * then bumps that rank's arrival counter; the merge kernel waits (bounded, 2 s, then
 * MF_ERR_TIMEOUT at mf_synchronize) until every rank's counter has reached the step's
 * expected value and merges out of its own memory.
 *   recv[r]     rank r's receive buffer, 2 * world * rows * (head_dim + 2) floats
 *               ([step parity][source rank][acc | m | l]), followed by the same blocks as 8-byte
 *               {tag, float} words (MF_OPTION_PUSH_TAGGED), mapped in this process
 *   counters[r] rank r's counters (8 per-source totals, 8 "merged by rank" counts, then one per
 *               unit), zero before the first step
 * Steps are numbered from 0 and must be issued in the same order on every rank, and a rank
 * pushes the same number of units in every step (the counters only ever grow: the value that
 * completes step s is units * (s + 1)).
 * Two step parities of receive blocks suffice between ranks that push: a rank's push of step
 * s + 2 follows its own merge of step s + 1, which waited for every other pusher's push of
 * s + 1, which that pusher's stream ordered after its merge of step s.  A rank that only merges
 * waits for nobody, so nothing in that chain holds the pushers back for it: such ranks are
 * named in merge_only_mask, they count every row they have merged on the pushers' "merged by"
 * words, and a pusher's decode kernel of step s >= 2 waits (bounded, 2 s, then a Timeout at
 * mf_synchronize) until each of them has merged step s - 2 before it overwrites that block. */
typedef struct MfPeerExchange {
    float *recv[8];
    uint32_t *counters[8];
    void *mapping[8]; /* what create / attach mapped; released by destroy */
    uint32_t world;
    uint32_t rank;
    uint32_t rows;     /* batch * n_heads, as given to create */
    uint32_t head_dim;
    uint32_t merge_only_mask; /* bit r: rank r never pushes, it only calls mf_merge_pushed (set by the
                               * caller, the same on every rank, before the first step; 0 after create) */
} MfPeerExchange;

#define MF_IPC_HANDLE_BYTES 64
/* Allocates this rank's buffers (zeroed), fills px for `rank`, and writes an inter-process
 * handle (MF_IPC_HANDLE_BYTES) that the other ranks pass to attach.  handle_out may be NULL
 * when world is 1.  The caller moves the handles between processes by its own means. */
MF_API mf_status mf_peer_exchange_create(MfContext *ctx, uint32_t world, uint32_t rank, uint32_t rows,
                                         uint32_t head_dim, MfPeerExchange *px, uint8_t *handle_out);
MF_API mf_status mf_peer_exchange_attach(MfContext *ctx, MfPeerExchange *px, uint32_t peer, const uint8_t *handle);
/* Every rank must have finished its last step (a host barrier) before any rank destroys. */
MF_API mf_status mf_peer_exchange_destroy(MfContext *ctx, MfPeerExchange *px);

MF_API mf_status mf_paged_decode_partial_push(MfContext *ctx, const MfDecodePlan *plan,
                                              const MfPagedKv *cache, const MfPagedDecodeArgs *args,
                                              const uint32_t *rope_positions, const MfPeerExchange *px,
                                              uint32_t step);
/* The same with the merge inside the decode kernel too: the CTA that finishes a (sequence, kv
 * head) unit pushes it, then waits (bounded) until every rank of pusher_mask (bit r = rank r
 * holds keys and runs this call in this step) has pushed that unit, merges the unit's query
 * heads out of local memory and writes args->out.  One launch per layer and rank, no second
 * kernel.  A rank that holds no keys cannot use this form (it has nothing to launch): it calls
 * mf_merge_pushed, and the ranks that do hold keys still push to it. */
MF_API mf_status mf_paged_decode_push_merge(MfContext *ctx, const MfDecodePlan *plan, const MfPagedKv *cache,
                                            const MfPagedDecodeArgs *args, const uint32_t *rope_positions,
                                            const MfPeerExchange *px, uint32_t step, uint32_t pusher_mask);
/* mf_paged_decode_partial_push over the 8-bit cache: the two-launch form (mf_merge_pushed merges, as for the f16
 * cache; the exchange object does not know which cache the partials came from). */
MF_API mf_status mf_paged_decode_kv8_partial_push(MfContext *ctx, const MfDecodePlan *plan, const MfPagedKv8 *cache,
                                                  const MfPagedDecodeArgs *args, const uint32_t *rope_positions,
                                                  const MfPeerExchange *px, uint32_t step);
/* mf_paged_decode_push_merge over the 8-bit cache (same exchange object, step numbering, pusher mask and wire
 * forms): one launch appends (quantising), attends over this shard's 8-bit pages, stores the unit's partial into
 * every rank's receive block and merges all ranks' partials into args->out.  No counterpart in the reference. */
MF_API mf_status mf_paged_decode_kv8_push_merge(MfContext *ctx, const MfDecodePlan *plan, const MfPagedKv8 *cache,
                                                const MfPagedDecodeArgs *args, const uint32_t *rope_positions,
                                                const MfPeerExchange *px, uint32_t step, uint32_t pusher_mask);
/* The same exchange through a library collective (the baseline the fused route is measured against,
 * and the route for hosts that already run NCCL): every rank passes its own block `mine` =
 * [acc rows*head_dim | m rows | l rows] f32 (what mf_paged_decode_partial wrote, laid out in one
 * buffer), the blocks of all ranks are all-gathered into `gathered` (world blocks) on the context's
 * stream with ncclAllGather on the caller's communicator `comm` (an ncclComm_t), and the log-sum-exp
 * merge of flash_prefill.metal:843-888 writes out [rows, head_dim] f16 on every rank.  The library
 * does not link NCCL: the symbol is taken from the process (or libnccl.so.2 is loaded) at first use;
 * MF_ERR_NCCL when it is not there or the collective returns an error. */
MF_API mf_status mf_allgather_merge(MfContext *ctx, void *comm, const float *mine, float *gathered, uint32_t world,
                                    uint32_t rows, uint32_t head_dim, void *out);
/* Replaces ncclAllGather in mf_allgather_merge by the caller's function (another collective library, a
 * statically linked NCCL, a test double): it gathers count_floats f32 per rank from send into recv on
 * `stream` and returns 0 on success.  NULL restores the default. */
typedef int (*MfAllGatherFn)(const void *send, void *recv, uint64_t count_floats, void *comm, void *stream);
MF_API mf_status mf_context_set_allgather(MfContext *ctx, MfAllGatherFn fn);

/* units_per_rank[r]: (batch x kv head) units rank r pushes per step (0 for a rank that
 * holds no keys); rows = batch * n_heads; out is [rows, head_dim] f16. */
MF_API mf_status mf_merge_pushed(MfContext *ctx, const MfPeerExchange *px, const uint32_t *units_per_rank,
                                 uint32_t step, uint32_t rows, uint32_t head_dim, void *out);

#ifdef __cplusplus
}
#endif
#endif /* METALLIC_CUDA_H */
