// What the append kernels and the two projection kernels share: a head row's chunk pair, its RoPE,
// the parameters of an append and the store of one rotated chunk pair (kv_append.cu has the
// kernels that use them on their own; fused_qkv_tc.cu is the tensor-core projection).
#pragma once
#include "internal.hpp"

namespace mf {

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
    uint32_t n_pages;            // paged: pages in the pool
    uint32_t *status;            // device status word (kStatusBadPage when a store was skipped)
    uint32_t rope_mode, apply_rope;
    uint32_t q_head_major;       // 1: q_rot is [Hq, M, D] (KvPrepFused); 0: [M, Hq*D]
};

// Rotate (unless V or RoPE is off) and store chunk pair j of head slot `slot` for input
// row s: the q slots go to q_rot, the k / v slots to the cache row of the token's position.
__device__ __forceinline__ void rope_and_store(const AppendParams &p, uint32_t s, uint32_t slot, uint32_t j,
                                               Chunk a, Chunk c)
{
    const uint32_t D = p.head_dim;
    uint32_t pos, b = 0;
    if (p.kv_lens && p.seq == 0xFFFFFFFFu) {
        b = s;  // one token per sequence
        const uint32_t len = p.kv_lens[b];
        if (len == 0) {  // nothing to append for an empty sequence; the table has no row for it
            atomicOr(p.status, kStatusBadPage);
            return;
        }
        pos = len - 1;
    } else {
        b = p.page_table ? p.seq : 0;
        pos = p.position_offset + s;
    }
    // The table and the lengths are the caller's device data: a position past the table or a page id
    // past the pool skips the access and raises the status bit instead of leaving the pool (the
    // reference's kernels return silently on a broken contract, flash_decode.metal:165-170).
    if (p.page_table && pos / p.page_size >= p.pt_stride) {
        atomicOr(p.status, kStatusBadPage);
        return;
    }
    const bool is_v = slot >= p.n_heads + p.n_kv_heads;
    if (p.apply_rope && !is_v) {
        const __half *cos_row = p.cos_t + (size_t)pos * (D / 2);
        const __half *sin_row = p.sin_t + (size_t)pos * (D / 2);
        rope_chunks(a, c, cos_row, sin_row, j, D, p.rope_mode);
    }
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
        if (page >= p.n_pages) {
            atomicOr(p.status, kStatusBadPage);
            return;
        }
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

struct QkvParams {
    const __half *x, *w_q, *w_k, *w_v, *gamma, *b_q, *b_k, *b_v;
    __half *out_q, *out_k, *out_v;
    uint32_t k_dim, n_dim, n_kv, m;
    uint32_t blocked;    // 1: element (r, k) at (k % 32) + 32 * (r + (k / 32) * N)
    uint32_t head_dim;   // rows per head slot (16 without the append)
    uint32_t q_slots, kv_slots;
    uint32_t rows_per_cta;  // input rows staged per CTA, at most 8
    float eps;
    uint32_t append;
    uint32_t strict_release;  // 1: dependents are released after the dependency wait, not at the start
};

// Projection of eight input rows or more on the tcgen05 tensor cores (fused_qkv_tc.cu).  Returns
// MF_ERR_OPERATION_NOT_SUPPORTED without launching anything when the shape is outside what it takes.
bool fused_qkv_tc_eligible(const MfContext *ctx, const QkvParams &qp);
mf_status launch_fused_qkv_tc(MfContext *ctx, QkvParams &qp, const AppendParams &ap, const char *what);

}  // namespace mf
