// RoPE + K/V append kernels (contiguous and paged caches) and the small
// rearrangement kernels of the reference's unfused chain.
//
// Replaces kv_prep_fused_kernel_f16 (kv_prep_fused.metal:26-123), rope_kernel_f16
// (rope.metal:28-75), kv_cache_write_kernel (kv_cache_write.metal:6-30),
// kv_cache_write_repeat_kv_heads_kernel (kv_cache_write_repeat.metal:9-40) and
// kv_cache_read_kernel (kv_cache_read.metal:7-29).  The reference launches one
// thread per f16 element and re-reads the RoPE mate and the cos/sin pair from
// device memory; here one thread owns two 16-byte chunks of a head row (chunk j
// and chunk j + D/16), so every global access is a 128-bit load or store and a
// NeoX pair (d, d + D/2) is rotated inside one thread.
//
// Rounding contract: operands widened f16 -> f32, x_i*c - x_j*s and x_j*c + x_i*s
// in f32 (both products are exact in f32, so contraction cannot change a bit),
// one round-to-nearest-even to f16.  V is a bit copy.
#include "internal.hpp"

namespace mf {
namespace {

union Chunk {
    uint4 u;
    __half h[8];
};

__device__ __forceinline__ __half rot_first(float xi, float xj, float c, float s)
{
    return __float2half_rn(__fsub_rn(__fmul_rn(xi, c), __fmul_rn(xj, s)));
}
__device__ __forceinline__ __half rot_second(float xi, float xj, float c, float s)
{
    return __float2half_rn(__fadd_rn(__fmul_rn(xj, c), __fmul_rn(xi, s)));
}

// Rotate chunks a = dims [8j, 8j+8) and b = dims [8j + D/2, 8j + D/2 + 8) of one
// head row in place.
__device__ __forceinline__ void rope_chunks(Chunk &a, Chunk &b, const __half *cos_row,
                                            const __half *sin_row, uint32_t j, uint32_t head_dim,
                                            uint32_t rope_mode)
{
    if (rope_mode == MF_ROPE_MODE_NEOX) {
        Chunk c, s;
        c.u = *reinterpret_cast<const uint4 *>(cos_row + 8 * j);
        s.u = *reinterpret_cast<const uint4 *>(sin_row + 8 * j);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float xi = __half2float(a.h[i]), xj = __half2float(b.h[i]);
            const float cv = __half2float(c.h[i]), sv = __half2float(s.h[i]);
            a.h[i] = rot_first(xi, xj, cv, sv);
            b.h[i] = rot_second(xi, xj, cv, sv);
        }
    } else {
        // adjacent pairs: dims (2i, 2i+1) use table entry i
        const uint32_t pa = 4 * j, pb = 4 * j + head_dim / 4;
        union {
            uint2 u;
            __half h[4];
        } ca, sa, cb, sb;
        ca.u = *reinterpret_cast<const uint2 *>(cos_row + pa);
        sa.u = *reinterpret_cast<const uint2 *>(sin_row + pa);
        cb.u = *reinterpret_cast<const uint2 *>(cos_row + pb);
        sb.u = *reinterpret_cast<const uint2 *>(sin_row + pb);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float xi = __half2float(a.h[2 * i]), xj = __half2float(a.h[2 * i + 1]);
            float cv = __half2float(ca.h[i]), sv = __half2float(sa.h[i]);
            a.h[2 * i] = rot_first(xi, xj, cv, sv);
            a.h[2 * i + 1] = rot_second(xi, xj, cv, sv);
            xi = __half2float(b.h[2 * i]);
            xj = __half2float(b.h[2 * i + 1]);
            cv = __half2float(cb.h[i]);
            sv = __half2float(sb.h[i]);
            b.h[2 * i] = rot_first(xi, xj, cv, sv);
            b.h[2 * i + 1] = rot_second(xi, xj, cv, sv);
        }
    }
}

struct AppendParams {
    const __half *q, *k, *v;
    __half *q_rot, *k_cache, *v_cache;
    const __half *cos_t, *sin_t;
    const uint32_t *page_table;  // null: contiguous cache
    const uint32_t *kv_lens;     // paged, one token per sequence
    uint32_t n_heads, n_kv_heads, head_dim, group;
    uint32_t seq_len;            // rows in q/k/v
    uint32_t position_offset;
    uint32_t max_seq_len;        // contiguous: cache capacity
    uint32_t cache_repeat;       // contiguous: 1 compact, G expanded
    uint32_t page_size, pt_stride, seq;  // paged
    uint32_t rope_mode, apply_rope;
    uint32_t q_head_major;       // 1: q_rot is [Hq, M, D] (KvPrepFused); 0: [M, Hq*D]
};

// One thread per (row s, head slot, chunk pair j).  Head slots: Hq query heads,
// then Hkv key heads, then Hkv value heads.
__global__ void __launch_bounds__(256) kv_append_kernel(const AppendParams p)
{
    const uint32_t cpr = p.head_dim / 16;  // chunk pairs per head row
    const uint32_t slots = p.n_heads + 2 * p.n_kv_heads;
    const uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t total = (uint64_t)p.seq_len * slots * cpr;
    if (gid >= total) return;
    const uint32_t j = gid % cpr;
    const uint32_t slot = (gid / cpr) % slots;
    const uint32_t s = gid / ((uint64_t)cpr * slots);
    const uint32_t D = p.head_dim;

    uint32_t pos, b = 0;
    if (p.kv_lens && p.seq == 0xFFFFFFFFu) {
        b = s;  // one token per sequence
        pos = p.kv_lens[b] - 1;
    } else {
        b = p.page_table ? p.seq : 0;
        pos = p.position_offset + s;
    }
    const __half *cos_row = p.cos_t + (size_t)pos * (D / 2);
    const __half *sin_row = p.sin_t + (size_t)pos * (D / 2);

    const __half *src;
    if (slot < p.n_heads)
        src = p.q + (size_t)s * p.n_heads * D + (size_t)slot * D;
    else if (slot < p.n_heads + p.n_kv_heads)
        src = p.k + (size_t)s * p.n_kv_heads * D + (size_t)(slot - p.n_heads) * D;
    else
        src = p.v + (size_t)s * p.n_kv_heads * D + (size_t)(slot - p.n_heads - p.n_kv_heads) * D;

    Chunk a, c;
    a.u = *reinterpret_cast<const uint4 *>(src + 8 * j);
    c.u = *reinterpret_cast<const uint4 *>(src + 8 * j + D / 2);
    const bool is_v = slot >= p.n_heads + p.n_kv_heads;
    if (p.apply_rope && !is_v) rope_chunks(a, c, cos_row, sin_row, j, D, p.rope_mode);

    if (slot < p.n_heads) {
        if (!p.q_rot) return;
        __half *dst = p.q_head_major ? p.q_rot + ((size_t)slot * p.seq_len + s) * D
                                     : p.q_rot + ((size_t)s * p.n_heads + slot) * D;
        *reinterpret_cast<uint4 *>(dst + 8 * j) = a.u;
        *reinterpret_cast<uint4 *>(dst + 8 * j + D / 2) = c.u;
        return;
    }
    const uint32_t kvh = is_v ? slot - p.n_heads - p.n_kv_heads : slot - p.n_heads;
    __half *cache = is_v ? p.v_cache : p.k_cache;
    if (p.page_table) {
        const uint32_t page = p.page_table[(size_t)b * p.pt_stride + pos / p.page_size];
        __half *dst = cache + (((size_t)page * p.n_kv_heads + kvh) * p.page_size + pos % p.page_size) * D;
        *reinterpret_cast<uint4 *>(dst + 8 * j) = a.u;
        *reinterpret_cast<uint4 *>(dst + 8 * j + D / 2) = c.u;
    } else {
        for (uint32_t g = 0; g < p.cache_repeat; ++g) {
            __half *dst = cache + ((size_t)(kvh * p.cache_repeat + g) * p.max_seq_len + pos) * D;
            *reinterpret_cast<uint4 *>(dst + 8 * j) = a.u;
            *reinterpret_cast<uint4 *>(dst + 8 * j + D / 2) = c.u;
        }
    }
}

// NeoX RoPE over rows of `dim` (rope.metal:36-74): pos = (row % seq_len) + offset.
__global__ void __launch_bounds__(256)
rope_kernel(const __half *in, __half *out, const __half *cos_t, const __half *sin_t, uint32_t dim,
            uint32_t seq_len, uint32_t position_offset, uint64_t rows)
{
    const uint32_t cpr = dim / 16;
    const uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= rows * cpr) return;
    const uint32_t j = gid % cpr;
    const uint64_t row = gid / cpr;
    const uint32_t pos = (uint32_t)(row % seq_len) + position_offset;
    Chunk a, c;
    a.u = *reinterpret_cast<const uint4 *>(in + row * dim + 8 * j);
    c.u = *reinterpret_cast<const uint4 *>(in + row * dim + 8 * j + dim / 2);
    rope_chunks(a, c, cos_t + (size_t)pos * (dim / 2), sin_t + (size_t)pos * (dim / 2), j, dim,
                MF_ROPE_MODE_NEOX);
    *reinterpret_cast<uint4 *>(out + row * dim + 8 * j) = a.u;
    *reinterpret_cast<uint4 *>(out + row * dim + 8 * j + dim / 2) = c.u;
}

// [H, M, D] -> rows position_offset..+M of a cache [H*repeat, cap, D], 16 bytes per thread.
__global__ void __launch_bounds__(256)
cache_write_kernel(const __half *in, __half *cache, uint32_t n_kv_heads, uint32_t head_dim, uint32_t m,
                   uint32_t position_offset, uint32_t max_seq_len, uint32_t repeat)
{
    const uint32_t cpr = head_dim / 8;
    const uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (uint64_t)n_kv_heads * m * cpr) return;
    const uint32_t j = gid % cpr;
    const uint32_t s = (gid / cpr) % m;
    const uint32_t h = gid / ((uint64_t)cpr * m);
    const uint4 x = *reinterpret_cast<const uint4 *>(in + ((size_t)h * m + s) * head_dim + 8 * j);
    for (uint32_t g = 0; g < repeat; ++g)
        *reinterpret_cast<uint4 *>(cache + ((size_t)(h * repeat + g) * max_seq_len + position_offset + s) * head_dim +
                                   8 * j) = x;
}

// cache [H, cap, D] -> [H, out_rows, D] rows [0, len); with a page table: pool -> rows of one sequence.
// out_rows == len packs the result (KvCacheRead); out_rows == a larger capacity re-strides the cache
// (growth: the head stride changes with the capacity, src/model/executor.rs:2493-2504).
__global__ void __launch_bounds__(256)
cache_read_kernel(const __half *cache, __half *out, uint32_t heads, uint32_t head_dim, uint32_t len,
                  uint32_t max_seq_len, const uint32_t *page_table_row, uint32_t page_size, uint32_t out_rows)
{
    const uint32_t cpr = head_dim / 8;
    const uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (uint64_t)heads * len * cpr) return;
    const uint32_t j = gid % cpr;
    const uint32_t t = (gid / cpr) % len;
    const uint32_t h = gid / ((uint64_t)cpr * len);
    const __half *src;
    if (page_table_row) {
        const uint32_t page = page_table_row[t / page_size];
        src = cache + (((size_t)page * heads + h) * page_size + t % page_size) * head_dim;
    } else {
        src = cache + ((size_t)h * max_seq_len + t) * head_dim;
    }
    *reinterpret_cast<uint4 *>(out + ((size_t)h * out_rows + t) * head_dim + 8 * j) =
        *reinterpret_cast<const uint4 *>(src + 8 * j);
}

// Contiguous cache rows [0, len) of every kv head -> the pages of one sequence (migration of a
// contiguous cache into the paged pool; the inverse of the paged read above).
__global__ void __launch_bounds__(256)
cache_to_pages_kernel(const __half *cache, __half *pool, uint32_t heads, uint32_t head_dim, uint32_t len,
                      uint32_t max_seq_len, const uint32_t *page_table_row, uint32_t page_size)
{
    const uint32_t cpr = head_dim / 8;
    const uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (uint64_t)heads * len * cpr) return;
    const uint32_t j = gid % cpr;
    const uint32_t t = (gid / cpr) % len;
    const uint32_t h = gid / ((uint64_t)cpr * len);
    const uint32_t page = page_table_row[t / page_size];
    __half *dst = pool + (((size_t)page * heads + h) * page_size + t % page_size) * head_dim;
    *reinterpret_cast<uint4 *>(dst + 8 * j) =
        *reinterpret_cast<const uint4 *>(cache + ((size_t)h * max_seq_len + t) * head_dim + 8 * j);
}

// kv_rearrange.metal:10-47 and repeat_kv_heads.metal:11-44: one thread per output element, same index
// arithmetic (the unfused chain is not on the hot path; the fused kernels never materialise these).
__global__ void __launch_bounds__(256)
kv_rearrange_kernel(const __half *__restrict__ in, __half *__restrict__ out, const KvRearrangeParamsResolved p)
{
    const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= p.total_elements) return;
    const uint32_t hd = gid % p.head_dim;
    const uint32_t tmp = gid / p.head_dim;
    const uint32_t s = tmp % p.seq;
    const uint32_t out_batch = tmp / p.seq;
    const uint32_t b = out_batch / p.n_heads, h = out_batch % p.n_heads;
    const uint32_t kv_h = h / (p.n_heads / p.n_kv_heads);
    const uint32_t base = kv_h * p.kv_head_dim + hd;
    if (base >= p.kv_dim) return;
    out[gid] = in[(size_t)(b * p.seq + s) * p.row_stride + base];
}

__global__ void __launch_bounds__(256)
repeat_kv_heads_kernel(const __half *__restrict__ in, __half *__restrict__ out, const RepeatKvHeadsParamsResolved p)
{
    const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= p.total_elements) return;
    const uint32_t d = gid % p.head_dim;
    const uint32_t tmp = gid / p.head_dim;
    const uint32_t s = tmp % p.seq;
    const uint32_t bh = tmp / p.seq;
    const uint32_t b = bh / p.n_heads, h = bh % p.n_heads;
    const uint32_t src_bh = b * p.n_kv_heads + h / p.group_size;
    out[gid] = in[((size_t)src_bh * p.cache_stride + s) * p.head_dim + d];
}

// Whole pages of both pools, dst_ids[i] <- src_ids[i]; one thread per 16 bytes.
__global__ void __launch_bounds__(256)
copy_pages_kernel(uint4 *k_pool, uint4 *v_pool, const uint32_t *__restrict__ src_ids, const uint32_t *__restrict__ dst_ids,
                  uint32_t n, uint64_t chunks_per_page)
{
    const uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (uint64_t)n * chunks_per_page * 2) return;
    const uint64_t c = gid % chunks_per_page;
    const uint64_t pi = gid / chunks_per_page;
    uint4 *pool = (pi & 1) ? v_pool : k_pool;
    const uint32_t i = (uint32_t)(pi >> 1);
    pool[(uint64_t)dst_ids[i] * chunks_per_page + c] = pool[(uint64_t)src_ids[i] * chunks_per_page + c];
}

inline uint32_t blocks_for(uint64_t threads) { return (uint32_t)((threads + 255) / 256); }

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace mf

using namespace mf;

extern "C" {

mf_status mf_kv_prep_fused(MfContext *ctx, const MfTensor *q, const MfTensor *k, const MfTensor *v,
                           const MfTensor *q_rot, const MfTensor *k_cache, const MfTensor *v_cache,
                           const MfTensor *cos, const MfTensor *sin, const KvPrepFusedParamsResolved *pr)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!pr) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "params");
    mf_status st;
    const MfTensor *ts[8] = {q, k, v, q_rot, k_cache, v_cache, cos, sin};
    const char *names[8] = {"q", "k", "v", "q_rot", "k_cache", "v_cache", "cos", "sin"};
    for (int i = 0; i < 8; ++i)
        if ((st = need_tensor(ctx, ts[i], names[i])) != MF_OK) return st;
    // Constraints stated on the reference kernel (kv_prep/mod.rs:149-156).
    if (pr->head_dim == 0 || pr->head_dim % 16 != 0)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "KvPrepFused: head_dim %u must be a multiple of 16", pr->head_dim);
    if (pr->n_kv_heads == 0 || pr->n_heads % pr->n_kv_heads != 0 || pr->group_size != pr->n_heads / pr->n_kv_heads)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "KvPrepFused: n_heads %u / n_kv_heads %u / group_size %u inconsistent",
                    pr->n_heads, pr->n_kv_heads, pr->group_size);
    if (pr->d_model != pr->n_heads * pr->head_dim || pr->kv_dim != pr->n_kv_heads * pr->head_dim)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "KvPrepFused: row stride must equal dim (d_model %u, kv_dim %u)",
                    pr->d_model, pr->kv_dim);
    if (pr->total_elements != pr->n_heads * pr->seq_len * pr->head_dim)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "KvPrepFused: total_elements %u != n_heads*seq_len*head_dim",
                    pr->total_elements);
    if ((uint64_t)pr->position_offset + pr->seq_len > pr->max_seq_len)
        return fail(ctx, MF_ERR_INVALID_OPERATION, "KvPrepFused: position_offset %u + seq_len %u exceeds max_seq_len %u",
                    pr->position_offset, pr->seq_len, pr->max_seq_len);
    if (pr->rope_mode > 1) return fail(ctx, MF_ERR_INVALID_OPERATION, "KvPrepFused: rope_mode %u", pr->rope_mode);
    if (k_cache->rank != 3 || v_cache->rank != 3 || k_cache->dims[1] != pr->max_seq_len ||
        k_cache->dims[2] != pr->head_dim || v_cache->dims[0] != k_cache->dims[0] ||
        v_cache->dims[1] != k_cache->dims[1] || v_cache->dims[2] != k_cache->dims[2])
        return fail(ctx, MF_ERR_INVALID_SHAPE, "KvPrepFused: caches must be rank-3 [heads, max_seq_len, head_dim]");
    uint32_t repeat;
    if (k_cache->dims[0] == pr->n_kv_heads)
        repeat = 1;
    else if (k_cache->dims[0] == pr->n_heads)
        repeat = pr->group_size;
    else
        return fail(ctx, MF_ERR_INVALID_SHAPE, "KV cache heads mismatch: got %llu, expected %u (expanded) or %u (compact)",
                    (unsigned long long)k_cache->dims[0], pr->n_heads, pr->n_kv_heads);
    if (pr->seq_len == 0) return MF_OK;
    AppendParams p{};
    p.q = tensor_ptr(q);
    p.k = tensor_ptr(k);
    p.v = tensor_ptr(v);
    p.q_rot = tensor_ptr(q_rot);
    p.k_cache = tensor_ptr(k_cache);
    p.v_cache = tensor_ptr(v_cache);
    p.cos_t = tensor_ptr(cos);
    p.sin_t = tensor_ptr(sin);
    const void *ptrs[8] = {p.q, p.k, p.v, p.q_rot, p.k_cache, p.v_cache, p.cos_t, p.sin_t};
    for (int i = 0; i < 8; ++i)
        if (!aligned16(ptrs[i])) return fail(ctx, MF_ERR_INVALID_SHAPE, "KvPrepFused: %s must be 16-byte aligned", names[i]);
    p.n_heads = pr->n_heads;
    p.n_kv_heads = pr->n_kv_heads;
    p.head_dim = pr->head_dim;
    p.group = pr->group_size;
    p.seq_len = pr->seq_len;
    p.position_offset = pr->position_offset;
    p.max_seq_len = pr->max_seq_len;
    p.cache_repeat = repeat;
    p.rope_mode = pr->rope_mode;
    // SmolLM3-style skip: no RoPE on every N-th layer (kv_prep_fused.metal:56-57).
    p.apply_rope = pr->no_rope_layer_step == 0 || ((pr->layer_idx + 1u) % pr->no_rope_layer_step) != 0u;
    p.q_head_major = 1;
    const uint64_t threads = (uint64_t)p.seq_len * (p.n_heads + 2 * p.n_kv_heads) * (p.head_dim / 16);
    kv_append_kernel<<<blocks_for(threads), 256, 0, ctx->stream>>>(p);
    return check_launch(ctx, "kv_append_kernel");
}

mf_status mf_paged_kv_append(MfContext *ctx, const MfPagedKv *cache, const void *q, const void *k, const void *v,
                             void *q_rot, const void *cos, const void *sin, uint32_t n_heads, uint32_t rope_mode,
                             uint32_t apply_rope, uint32_t seq, uint32_t position_offset, uint32_t seq_len)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!cache || !cache->k_pool || !cache->v_pool || !cache->page_table || !q || !k || !v)
        return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged append: null input");
    if (apply_rope && (!cos || !sin)) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged append: cos/sin");
    if (cache->head_dim % 16 != 0 || cache->n_kv_heads == 0 || n_heads % cache->n_kv_heads != 0)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "paged append: geometry");
    if (rope_mode > 1) return fail(ctx, MF_ERR_INVALID_OPERATION, "paged append: rope_mode %u", rope_mode);
    AppendParams p{};
    p.q = static_cast<const __half *>(q);
    p.k = static_cast<const __half *>(k);
    p.v = static_cast<const __half *>(v);
    p.q_rot = static_cast<__half *>(q_rot);
    p.k_cache = static_cast<__half *>(cache->k_pool);
    p.v_cache = static_cast<__half *>(cache->v_pool);
    p.cos_t = static_cast<const __half *>(cos);
    p.sin_t = static_cast<const __half *>(sin);
    p.page_table = cache->page_table;
    p.n_heads = n_heads;
    p.n_kv_heads = cache->n_kv_heads;
    p.head_dim = cache->head_dim;
    p.group = n_heads / cache->n_kv_heads;
    p.page_size = cache->page_size;
    p.pt_stride = cache->page_table_stride;
    p.rope_mode = rope_mode;
    p.apply_rope = apply_rope;
    p.seq = seq;
    if (seq == 0xFFFFFFFFu) {
        if (!cache->kv_lens) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged append: kv_lens");
        p.kv_lens = cache->kv_lens;
        p.seq_len = cache->batch;
        p.q_head_major = 0;
    } else {
        if (seq >= cache->batch) return fail(ctx, MF_ERR_INVALID_OPERATION, "paged append: sequence %u of %u", seq, cache->batch);
        if (((uint64_t)position_offset + seq_len + cache->page_size - 1) / cache->page_size > cache->page_table_stride)
            return fail(ctx, MF_ERR_INVALID_OPERATION, "paged append: rows %u..%u exceed the page table", position_offset,
                        position_offset + seq_len);
        p.seq_len = seq_len;
        p.position_offset = position_offset;
        p.q_head_major = 1;
    }
    if (p.seq_len == 0) return MF_OK;
    const uint64_t threads = (uint64_t)p.seq_len * (p.n_heads + 2 * p.n_kv_heads) * (p.head_dim / 16);
    kv_append_kernel<<<blocks_for(threads), 256, 0, ctx->stream>>>(p);
    return check_launch(ctx, "kv_append_kernel(paged)");
}

mf_status mf_rope(MfContext *ctx, const MfTensor *input, const MfTensor *output, const MfTensor *cos,
                  const MfTensor *sin, const RopeParamsResolved *pr)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!pr) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "params");
    mf_status st;
    if ((st = need_tensor(ctx, input, "input")) != MF_OK) return st;
    if ((st = need_tensor(ctx, output, "output")) != MF_OK) return st;
    if ((st = need_tensor(ctx, cos, "cos")) != MF_OK) return st;
    if ((st = need_tensor(ctx, sin, "sin")) != MF_OK) return st;
    if (pr->dim == 0 || pr->dim % 16 != 0 || pr->seq_len == 0 || pr->total_elements % pr->dim != 0)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "Rope: dim %u seq_len %u total %u", pr->dim, pr->seq_len,
                    pr->total_elements);
    const uint64_t rows = pr->total_elements / pr->dim;
    if (rows == 0) return MF_OK;
    rope_kernel<<<blocks_for(rows * (pr->dim / 16)), 256, 0, ctx->stream>>>(
        tensor_ptr(input), tensor_ptr(output), tensor_ptr(cos), tensor_ptr(sin), pr->dim, pr->seq_len,
        pr->position_offset, rows);
    return check_launch(ctx, "rope_kernel");
}

static mf_status cache_write_common(MfContext *ctx, const MfTensor *input, const MfTensor *cache, uint32_t n_kv_heads,
                                    uint32_t head_dim, uint32_t m, uint32_t position_offset, uint32_t max_seq_len,
                                    uint32_t repeat)
{
    mf_status st;
    if ((st = need_tensor(ctx, input, "input")) != MF_OK) return st;
    if ((st = need_tensor(ctx, cache, "cache")) != MF_OK) return st;
    if (head_dim == 0 || head_dim % 8 != 0) return fail(ctx, MF_ERR_INVALID_SHAPE, "KvCacheWrite: head_dim %u", head_dim);
    if ((uint64_t)position_offset + m > max_seq_len)
        return fail(ctx, MF_ERR_INVALID_OPERATION, "KvCacheWrite: position_offset %u + %u exceeds max_seq_len %u",
                    position_offset, m, max_seq_len);
    if (m == 0 || n_kv_heads == 0) return MF_OK;
    cache_write_kernel<<<blocks_for((uint64_t)n_kv_heads * m * (head_dim / 8)), 256, 0, ctx->stream>>>(
        tensor_ptr(input), tensor_ptr(cache), n_kv_heads, head_dim, m, position_offset, max_seq_len, repeat);
    return check_launch(ctx, "cache_write_kernel");
}

mf_status mf_kv_cache_write(MfContext *ctx, const MfTensor *input, const MfTensor *cache,
                            const KvCacheWriteParamsResolved *pr)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!pr) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "params");
    return cache_write_common(ctx, input, cache, pr->n_kv_heads, pr->head_dim, pr->input_seq_len, pr->position_offset,
                              pr->max_seq_len, 1);
}

mf_status mf_kv_cache_write_repeat_kv_heads(MfContext *ctx, const MfTensor *input, const MfTensor *cache,
                                            const KvCacheWriteRepeatKvHeadsParamsResolved *pr)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!pr) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "params");
    if (pr->n_kv_heads == 0 || pr->group_size == 0 || pr->n_heads != pr->n_kv_heads * pr->group_size)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "KvCacheWriteRepeatKvHeads: n_heads %u != n_kv_heads %u * group_size %u",
                    pr->n_heads, pr->n_kv_heads, pr->group_size);
    return cache_write_common(ctx, input, cache, pr->n_kv_heads, pr->head_dim, pr->input_seq_len, pr->position_offset,
                              pr->max_seq_len, pr->group_size);
}

mf_status mf_kv_cache_read(MfContext *ctx, const MfTensor *cache, const MfTensor *output, uint32_t seq_len)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    mf_status st;
    if ((st = need_tensor(ctx, cache, "cache")) != MF_OK) return st;
    if ((st = need_tensor(ctx, output, "output")) != MF_OK) return st;
    if (cache->rank != 3) return fail(ctx, MF_ERR_INVALID_SHAPE, "KvCacheRead: cache must be rank-3");
    if (seq_len > cache->dims[1]) return fail(ctx, MF_ERR_INVALID_OPERATION, "KvCacheRead: seq_len %u > capacity", seq_len);
    if (cache->dims[2] % 8 != 0) return fail(ctx, MF_ERR_INVALID_SHAPE, "KvCacheRead: head_dim");
    if (seq_len == 0) return MF_OK;
    const uint32_t heads = (uint32_t)cache->dims[0], hd = (uint32_t)cache->dims[2];
    cache_read_kernel<<<blocks_for((uint64_t)heads * seq_len * (hd / 8)), 256, 0, ctx->stream>>>(
        tensor_ptr(cache), tensor_ptr(output), heads, hd, seq_len, (uint32_t)cache->dims[1], nullptr, 0, seq_len);
    return check_launch(ctx, "cache_read_kernel");
}

// reallocate_kv_buffers / preserve_kv_cache (src/model/executor.rs:2437-2513).
mf_status mf_kv_cache_grow(MfContext *ctx, const MfTensor *old_cache, const MfTensor *new_cache, uint32_t current_pos)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    mf_status st;
    if ((st = need_tensor(ctx, old_cache, "old cache")) != MF_OK) return st;
    if ((st = need_tensor(ctx, new_cache, "new cache")) != MF_OK) return st;
    if (old_cache->rank != 3 || new_cache->rank != 3)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "KV cache tensor must be rank-3 [heads, seq, head_dim]");
    if (old_cache->dims[0] != new_cache->dims[0])
        return fail(ctx, MF_ERR_INVALID_SHAPE, "KV cache layout changed during growth: old heads=%llu, new heads=%llu",
                    (unsigned long long)old_cache->dims[0], (unsigned long long)new_cache->dims[0]);
    if (old_cache->dims[2] != new_cache->dims[2] || old_cache->dims[2] % 8 != 0)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "KV cache head_dim mismatch during growth");
    if (current_pos > old_cache->dims[1] || current_pos > new_cache->dims[1])
        return fail(ctx, MF_ERR_INVALID_OPERATION, "KV growth: %u tokens do not fit capacities %llu -> %llu", current_pos,
                    (unsigned long long)old_cache->dims[1], (unsigned long long)new_cache->dims[1]);
    if (current_pos == 0) return MF_OK;
    const uint32_t heads = (uint32_t)old_cache->dims[0], hd = (uint32_t)old_cache->dims[2];
    cache_read_kernel<<<blocks_for((uint64_t)heads * current_pos * (hd / 8)), 256, 0, ctx->stream>>>(
        tensor_ptr(old_cache), tensor_ptr(new_cache), heads, hd, current_pos, (uint32_t)old_cache->dims[1], nullptr, 0,
        (uint32_t)new_cache->dims[1]);
    return check_launch(ctx, "cache_read_kernel(grow)");
}

mf_status mf_kv_cache_to_pages(MfContext *ctx, const MfTensor *cache, const MfPagedKv *paged, uint32_t use_v, uint32_t seq,
                               uint32_t len)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    mf_status st;
    if ((st = need_tensor(ctx, cache, "cache")) != MF_OK) return st;
    if (!paged || !paged->k_pool || !paged->v_pool || !paged->page_table)
        return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "cache to pages: null input");
    if (cache->rank != 3 || cache->dims[0] != paged->n_kv_heads || cache->dims[2] != paged->head_dim)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "cache to pages: the cache must be compact [n_kv_heads, capacity, head_dim]");
    if (seq >= paged->batch) return fail(ctx, MF_ERR_INVALID_OPERATION, "cache to pages: sequence %u of %u", seq, paged->batch);
    if (len > cache->dims[1] || ((uint64_t)len + paged->page_size - 1) / paged->page_size > paged->page_table_stride)
        return fail(ctx, MF_ERR_INVALID_OPERATION, "cache to pages: %u tokens exceed the cache or the page table", len);
    if (len == 0) return MF_OK;
    __half *pool = static_cast<__half *>(use_v ? paged->v_pool : paged->k_pool);
    cache_to_pages_kernel<<<blocks_for((uint64_t)paged->n_kv_heads * len * (paged->head_dim / 8)), 256, 0, ctx->stream>>>(
        tensor_ptr(cache), pool, paged->n_kv_heads, paged->head_dim, len, (uint32_t)cache->dims[1],
        paged->page_table + (size_t)seq * paged->page_table_stride, paged->page_size);
    return check_launch(ctx, "cache_to_pages_kernel");
}

mf_status mf_kv_rearrange(MfContext *ctx, const MfTensor *input, const MfTensor *output, const KvRearrangeParamsResolved *p)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    mf_status st;
    if ((st = need_tensor(ctx, input, "input")) != MF_OK) return st;
    if ((st = need_tensor(ctx, output, "output")) != MF_OK) return st;
    if (!p) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "KvRearrange: params");
    if (p->total_elements == 0) return MF_OK;
    if (p->n_kv_heads == 0 || p->n_heads % p->n_kv_heads != 0 || p->head_dim == 0 || p->seq == 0)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "KvRearrange: n_heads %u, n_kv_heads %u, head_dim %u, seq %u", p->n_heads,
                    p->n_kv_heads, p->head_dim, p->seq);
    kv_rearrange_kernel<<<blocks_for(p->total_elements), 256, 0, ctx->stream>>>(tensor_ptr(input), tensor_ptr(output), *p);
    return check_launch(ctx, "kv_rearrange_kernel");
}

mf_status mf_repeat_kv_heads(MfContext *ctx, const MfTensor *input, const MfTensor *output,
                             const RepeatKvHeadsParamsResolved *p)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    mf_status st;
    if ((st = need_tensor(ctx, input, "input")) != MF_OK) return st;
    if ((st = need_tensor(ctx, output, "output")) != MF_OK) return st;
    if (!p) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "RepeatKvHeads: params");
    if (p->total_elements == 0) return MF_OK;
    if (p->group_size == 0 || p->n_heads != p->n_kv_heads * p->group_size || p->head_dim == 0 || p->seq == 0 ||
        p->seq > p->cache_stride)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "RepeatKvHeads: n_heads %u, n_kv_heads %u, group %u, seq %u, cache_stride %u",
                    p->n_heads, p->n_kv_heads, p->group_size, p->seq, p->cache_stride);
    repeat_kv_heads_kernel<<<blocks_for(p->total_elements), 256, 0, ctx->stream>>>(tensor_ptr(input), tensor_ptr(output), *p);
    return check_launch(ctx, "repeat_kv_heads_kernel");
}

mf_status mf_paged_copy_pages(MfContext *ctx, const MfPagedKv *cache, const uint32_t *src_ids, const uint32_t *dst_ids,
                              uint32_t n)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!cache || !cache->k_pool || !cache->v_pool || (n && (!src_ids || !dst_ids)))
        return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "copy pages: null input");
    if (n == 0) return MF_OK;
    const uint64_t chunks = (uint64_t)cache->n_kv_heads * cache->page_size * (cache->head_dim / 8);  // 16-byte units per page
    copy_pages_kernel<<<blocks_for((uint64_t)n * chunks * 2), 256, 0, ctx->stream>>>(
        static_cast<uint4 *>(cache->k_pool), static_cast<uint4 *>(cache->v_pool), src_ids, dst_ids, n, chunks);
    return check_launch(ctx, "copy_pages_kernel");
}

mf_status mf_paged_gather(MfContext *ctx, const MfPagedKv *cache, uint32_t use_v, uint32_t seq, uint32_t len, void *out)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!cache || !cache->k_pool || !cache->v_pool || !cache->page_table || !out)
        return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged gather: null input");
    if (seq >= cache->batch) return fail(ctx, MF_ERR_INVALID_OPERATION, "paged gather: sequence %u of %u", seq, cache->batch);
    if (((uint64_t)len + cache->page_size - 1) / cache->page_size > cache->page_table_stride)
        return fail(ctx, MF_ERR_INVALID_OPERATION, "paged gather: %u tokens exceed the page table", len);
    if (len == 0) return MF_OK;
    const __half *pool = static_cast<const __half *>(use_v ? cache->v_pool : cache->k_pool);
    cache_read_kernel<<<blocks_for((uint64_t)cache->n_kv_heads * len * (cache->head_dim / 8)), 256, 0, ctx->stream>>>(
        pool, static_cast<__half *>(out), cache->n_kv_heads, cache->head_dim, len, 0,
        cache->page_table + (size_t)seq * cache->page_table_stride, cache->page_size, len);
    return check_launch(ctx, "cache_read_kernel(paged)");
}

}  // extern "C"
