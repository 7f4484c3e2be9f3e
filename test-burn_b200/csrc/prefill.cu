// Causal chunked prefill attention over the contiguous F16 KV cache (M > 1).
//
// Replaces flash_prefill_tiled_d64/d128 (flash_prefill.metal:94-446) and the
// split-K pair flash_prefill_splitk_part / _reduce (:460-983).  Contract kept:
// key k is visible to query row r iff k <= r + query_offset; scores are f16 x f16
// products accumulated in f32 times `scale`; masked scores are -1e30 and the
// running max starts there; weights, l and the accumulator are f32; the result is
// acc * (1/l) or 0 when l is not finite or <= 1e-6; rows >= q_len are not written;
// split-K partials are unnormalised f32 (acc, m, l) merged with the log-sum-exp
// rule.  The reference computes every dot product with SIMD-group sums and visits
// fully masked tiles; this kernel puts QK^T and PV on tensor cores and stops at
// the causal diagonal.
//
// This file is the mma.sync (m16n8k16) implementation: one CTA per (64-row query
// tile, query head, split); a producer warp streams 64-key K/V tiles with TMA
// into a shared-memory ring (128-byte swizzle), four consumer warps own 16 query
// rows each.
#include <algorithm>

#include "internal.hpp"
#include "ptx.cuh"

namespace mf {
namespace {

constexpr uint32_t kPfWarps = 4;
constexpr uint32_t kPfThreads = kPfWarps * 32 + 32;
constexpr uint32_t kPfTileM = 16 * kPfWarps;
constexpr float kNeg = -1e30f;
constexpr uint64_t kPfWaitNs = 2000000000ull;

struct PrefillParams {
    const __half *q;
    __half *out;
    float *part_acc, *part_m, *part_l;  // split-K scratch or null
    uint32_t *status;
    uint32_t q_len, kv_len, query_offset, group;
    uint32_t q_stride_h, q_stride_m, out_stride_h, out_stride_m;
    uint32_t k_rows_h, v_rows_h;  // cache rows per head
    uint32_t n_heads, split_k, keys_per_split;
    float scale_log2;
    // Paged cache: the sequence's page ids (device), tokens per page, kv heads; null for a contiguous cache.
    const uint32_t *page_table_row;
    uint32_t page_size, n_kv_heads;
};

__device__ __forceinline__ uint32_t pf_tile_off(uint32_t row, uint32_t c16)
{
    return (c16 >> 3) * (kTileKeys * 128) + row * 128 + (((c16 & 7) ^ (row & 7)) << 4);
}

template <int D, int STAGES>
__global__ void __launch_bounds__(kPfThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
               const PrefillParams p)
{
    constexpr uint32_t kTileBytes = kTileKeys * D * 2;
    constexpr uint32_t kStageBytes = 2 * kTileBytes;
    constexpr uint32_t kHalfBytes = kTileKeys * 128;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_full = smem_base + STAGES * kStageBytes;
    const uint32_t bar_empty = bar_full + STAGES * 8;
    volatile uint32_t *abort_flag =
        reinterpret_cast<volatile uint32_t *>(smem_raw + (smem_base - smem_u32(smem_raw)) + STAGES * kStageBytes + 2 * STAGES * 8);

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Heavy (late) query tiles first so the causal tail does not end the grid.
    const uint32_t q_tile = gridDim.x - 1 - blockIdx.x;
    const uint32_t head = blockIdx.y;
    const uint32_t split = blockIdx.z;
    const uint32_t kvh = head / p.group;
    const uint32_t row0 = q_tile * kPfTileM;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, kPfWarps);
        }
        *abort_flag = 0;
        mbar_fence_init();
        fence_proxy_async();
    }
    __syncthreads();

    // Key range of this CTA: its split's range, cut at the causal limit of the tile's last row.
    uint32_t key_begin = split * p.keys_per_split;
    uint32_t key_end = min(p.kv_len, key_begin + p.keys_per_split);
    const uint32_t last_row = min(p.q_len, row0 + kPfTileM) - 1;
    key_end = min(key_end, last_row + p.query_offset + 1);
    const uint32_t tile_begin = key_begin / kTileKeys;
    const uint32_t tile_end = key_end > key_begin ? (key_end + kTileKeys - 1) / kTileKeys : tile_begin;

    if (warp == kPfWarps) {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, issued = 0;
            for (uint32_t t = tile_begin; t < tile_end; ++t) {
                if (!*abort_flag && !mbar_wait_bounded(bar_empty + stage * 8, phase ^ 1, kPfWaitNs)) {
                    *abort_flag = 1;
                    atomicOr(p.status, 4u);
                }
                const uint32_t full = bar_full + stage * 8;
                const uint32_t dst_k = smem_base + stage * kStageBytes, dst_v = dst_k + kTileBytes;
                if (p.page_table_row) {
                    // one box per page (or per 64 rows of a larger page) and 64-column half; pages past the
                    // last key are not fetched: their rows are masked, and cleared in V, by the consumers
                    const uint32_t rpb = min(p.page_size, kTileKeys), n_box = kTileKeys / rpb;
                    uint32_t live = 0;
                    for (uint32_t j = 0; j < n_box; ++j) live += (t * kTileKeys + j * rpb < p.kv_len) ? 1u : 0u;
                    mbar_arrive_expect_tx(full, live * rpb * D * 4);
                    for (uint32_t j = 0; j < live; ++j) {
                        const uint32_t tok = t * kTileKeys + j * rpb;
                        const uint32_t page = __ldg(p.page_table_row + tok / p.page_size);
                        const int32_t r = (int32_t)((page * p.n_kv_heads + kvh) * p.page_size + tok % p.page_size);
#pragma unroll
                        for (int h = 0; h < D / 64; ++h) {
                            tma_load_2d(dst_k + h * kHalfBytes + j * rpb * 128, &tm_k, h * 64, r, full);
                            tma_load_2d(dst_v + h * kHalfBytes + j * rpb * 128, &tm_v, h * 64, r, full);
                        }
                    }
                } else {
                    mbar_arrive_expect_tx(full, kStageBytes);
                    const int32_t rk = (int32_t)(kvh * p.k_rows_h + t * kTileKeys);
                    const int32_t rv = (int32_t)(kvh * p.v_rows_h + t * kTileKeys);
#pragma unroll
                    for (int h = 0; h < D / 64; ++h) {
                        tma_load_2d(dst_k + h * kHalfBytes, &tm_k, h * 64, rk, full);
                        tma_load_2d(dst_v + h * kHalfBytes, &tm_v, h * 64, rv, full);
                    }
                }
                ++issued;
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (*abort_flag) {
                const uint32_t n = issued < (uint32_t)STAGES ? issued : (uint32_t)STAGES;
                for (uint32_t i = 0; i < n; ++i) {
                    const uint32_t s = (stage + STAGES - 1 - i) % STAGES;
                    (void)mbar_wait_bounded(bar_full + s * 8, (s < stage) ? phase : (phase ^ 1), kPfWaitNs);
                }
            }
        }
        return;
    }

    // ---- consumers: 16 query rows per warp ------------------------------------------
    const uint32_t r_lo = row0 + warp * 16 + (lane >> 2);  // rows of c0/c1; c2/c3 are r_lo + 8
    const uint32_t r_hi = r_lo + 8;
    const bool ok_lo = r_lo < p.q_len, ok_hi = r_hi < p.q_len;

    // A fragments of Q (16 rows x D), straight from global memory.
    uint32_t aq[D / 16][4];
    {
        const __half *q_lo = p.q + (size_t)head * p.q_stride_h + (size_t)r_lo * p.q_stride_m + 2 * (lane & 3);
        const __half *q_hi = q_lo + (size_t)8 * p.q_stride_m;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            aq[ks][0] = ok_lo ? *reinterpret_cast<const uint32_t *>(q_lo + ks * 16) : 0u;
            aq[ks][1] = ok_hi ? *reinterpret_cast<const uint32_t *>(q_hi + ks * 16) : 0u;
            aq[ks][2] = ok_lo ? *reinterpret_cast<const uint32_t *>(q_lo + ks * 16 + 8) : 0u;
            aq[ks][3] = ok_hi ? *reinterpret_cast<const uint32_t *>(q_hi + ks * 16 + 8) : 0u;
        }
    }
    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m_lo = kNeg, m_hi = kNeg, l_lo = 0.f, l_hi = 0.f;
    const uint32_t lim_lo = r_lo + p.query_offset, lim_hi = r_hi + p.query_offset;
    const uint32_t warp_last_row = row0 + warp * 16 + 15;

    uint32_t stage = 0, phase = 0;
    for (uint32_t t = tile_begin; t < tile_end; ++t) {
        if (!*abort_flag && !mbar_wait_bounded(bar_full + stage * 8, phase, kPfWaitNs)) {
            *abort_flag = 1;
            atomicOr(p.status, 8u);
        }
        const uint32_t k_addr = smem_base + stage * kStageBytes, v_addr = k_addr + kTileBytes;
        const uint32_t key0 = t * kTileKeys;
        if (t + 1 == tile_end && key_end < key0 + kTileKeys) {
            // Rows past the last visible key may never have been written (capacity slack):
            // clear them in V so that a zero weight cannot meet a NaN.
            uint8_t *v_tile = smem_raw + (smem_base - smem_u32(smem_raw)) + stage * kStageBytes + kTileBytes;
            const uint32_t first_dead = key_end - key0;
            const uint32_t n_chunks = (kTileKeys - first_dead) * (D / 8);
            for (uint32_t c = tid; c < n_chunks; c += kPfWarps * 32) {
                const uint32_t row = first_dead + c / (D / 8);
                *reinterpret_cast<uint4 *>(v_tile + pf_tile_off(row, c % (D / 8))) = make_uint4(0, 0, 0, 0);
            }
            fence_proxy_async();
            named_bar_sync(1, kPfWarps * 32);
        }
        // Skip tiles wholly above this warp's causal limit.
        if (key0 <= warp_last_row + p.query_offset) {
            float c[8][4];
#pragma unroll
            for (int n = 0; n < 8; ++n) c[n][0] = c[n][1] = c[n][2] = c[n][3] = 0.f;
            // S (16 rows x 64 keys) = Q K^T.  B fragments (k = dims, n = keys) come from
            // K rows with a plain ldmatrix: x4 covers 16 keys x 16 dims = two n-tiles.
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t b[4];
                    const uint32_t row = np * 16 + (lane & 7) + (lane >> 4) * 8;
                    ldmatrix_x4(b, k_addr + pf_tile_off(row, 2 * ks + ((lane >> 3) & 1)));
                    mma_m16n8k16(c[2 * np], aq[ks], b[0], b[1]);
                    mma_m16n8k16(c[2 * np + 1], aq[ks], b[2], b[3]);
                }
            }
            // scale, mask, row max
            const bool need_mask = (key0 + kTileKeys - 1 > r_lo + p.query_offset) || (key0 < key_begin) ||
                                   (key0 + kTileKeys > key_end);
            float mx_lo = kNeg, mx_hi = kNeg;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float s = c[n][e] * p.scale_log2;
                    if (!(fabsf(s) <= 3.0e38f)) s = kNeg;
                    if (need_mask) {
                        const uint32_t key = key0 + n * 8 + 2 * (lane & 3) + (e & 1);
                        const uint32_t lim = (e & 2) ? lim_hi : lim_lo;
                        if (key > lim || key < key_begin || key >= key_end) s = kNeg;
                    }
                    c[n][e] = s;
                }
                mx_lo = fmaxf(mx_lo, fmaxf(c[n][0], c[n][1]));
                mx_hi = fmaxf(mx_hi, fmaxf(c[n][2], c[n][3]));
            }
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
            const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
            const float a_lo = fast_exp2(m_lo - mn_lo), a_hi = fast_exp2(m_hi - mn_hi);
            m_lo = mn_lo;
            m_hi = mn_hi;
            float s_lo = 0.f, s_hi = 0.f;
            uint32_t pa[4][4];  // A fragments of P for the 4 k-steps of 16 keys
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                // A masked score is exactly the sentinel; its weight is 0 even when the row
                // has seen nothing but masked keys so far (then s - m would be 0).
                const float p0 = c[n][0] == kNeg ? 0.f : fast_exp2(c[n][0] - mn_lo);
                const float p1 = c[n][1] == kNeg ? 0.f : fast_exp2(c[n][1] - mn_lo);
                const float p2 = c[n][2] == kNeg ? 0.f : fast_exp2(c[n][2] - mn_hi);
                const float p3 = c[n][3] == kNeg ? 0.f : fast_exp2(c[n][3] - mn_hi);
                s_lo += p0 + p1;
                s_hi += p2 + p3;
                pa[n >> 1][(n & 1) * 2] = pack_f16x2(p0, p1);
                pa[n >> 1][(n & 1) * 2 + 1] = pack_f16x2(p2, p3);
            }
            l_lo = l_lo * a_lo + s_lo;
            l_hi = l_hi * a_hi + s_hi;
#pragma unroll
            for (int n = 0; n < D / 8; ++n) {
                o[n][0] *= a_lo;
                o[n][1] *= a_lo;
                o[n][2] *= a_hi;
                o[n][3] *= a_hi;
            }
            // O (16 rows x D) += P V.  B fragments (k = keys, n = dims) from V rows with a
            // transposing ldmatrix: x4 covers 16 keys x 16 dims = two n-tiles.
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                for (int dp = 0; dp < D / 16; ++dp) {
                    uint32_t b[4];
                    const uint32_t row = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4_trans(b, v_addr + pf_tile_off(row, 2 * dp + (lane >> 4)));
                    mma_m16n8k16(o[2 * dp], pa[kk], b[0], b[1]);
                    mma_m16n8k16(o[2 * dp + 1], pa[kk], b[2], b[3]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + stage * 8);
        if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
        }
    }

    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

    if (p.part_acc) {
        // Unnormalised partials, [split][head][row] order.
        const size_t base = ((size_t)split * p.n_heads + head) * p.q_len;
        if (ok_lo) {
            float *dst = p.part_acc + (base + r_lo) * D + 2 * (lane & 3);
#pragma unroll
            for (int n = 0; n < D / 8; ++n) *reinterpret_cast<float2 *>(dst + n * 8) = make_float2(o[n][0], o[n][1]);
            if ((lane & 3) == 0) {
                p.part_m[base + r_lo] = m_lo * 0.6931471805599453f;
                p.part_l[base + r_lo] = l_lo;
            }
        }
        if (ok_hi) {
            float *dst = p.part_acc + (base + r_hi) * D + 2 * (lane & 3);
#pragma unroll
            for (int n = 0; n < D / 8; ++n) *reinterpret_cast<float2 *>(dst + n * 8) = make_float2(o[n][2], o[n][3]);
            if ((lane & 3) == 0) {
                p.part_m[base + r_hi] = m_hi * 0.6931471805599453f;
                p.part_l[base + r_hi] = l_hi;
            }
        }
        return;
    }
    const float inv_lo = ((fabsf(l_lo) <= 3.0e38f) && fabsf(l_lo) > 1e-6f) ? 1.0f / l_lo : 0.f;
    const float inv_hi = ((fabsf(l_hi) <= 3.0e38f) && fabsf(l_hi) > 1e-6f) ? 1.0f / l_hi : 0.f;
    if (ok_lo) {
        __half *dst = p.out + (size_t)r_lo * p.out_stride_m + (size_t)head * p.out_stride_h + 2 * (lane & 3);
#pragma unroll
        for (int n = 0; n < D / 8; ++n)
            *reinterpret_cast<__half2 *>(dst + n * 8) = __floats2half2_rn(o[n][0] * inv_lo, o[n][1] * inv_lo);
    }
    if (ok_hi) {
        __half *dst = p.out + (size_t)r_hi * p.out_stride_m + (size_t)head * p.out_stride_h + 2 * (lane & 3);
#pragma unroll
        for (int n = 0; n < D / 8; ++n)
            *reinterpret_cast<__half2 *>(dst + n * 8) = __floats2half2_rn(o[n][2] * inv_hi, o[n][3] * inv_hi);
    }
}

// Split-K reduce writing token-major output (flash_prefill.metal:806-983).
__global__ void __launch_bounds__(128)
prefill_reduce_kernel(const float *__restrict__ acc, const float *__restrict__ m, const float *__restrict__ l,
                      uint32_t split_k, uint32_t n_heads, uint32_t q_len, uint32_t head_dim, __half *__restrict__ out,
                      uint32_t out_stride_h, uint32_t out_stride_m)
{
    const uint32_t row = blockIdx.x, head = blockIdx.y;
    const size_t rows = (size_t)n_heads * q_len;
    const size_t idx = (size_t)head * q_len + row;
    float mx = -1e30f;
    for (uint32_t s = 0; s < split_k; ++s) mx = fmaxf(mx, m[s * rows + idx]);
    float lt = 0.f;
    for (uint32_t s = 0; s < split_k; ++s) {
        const float ls = l[s * rows + idx];
        if (ls > 0.f) lt += ls * __expf(m[s * rows + idx] - mx);
    }
    const float inv = ((fabsf(lt) <= 3.0e38f) && fabsf(lt) > 1e-6f) ? 1.0f / lt : 0.f;
    for (uint32_t d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float a = 0.f;
        for (uint32_t s = 0; s < split_k; ++s) a += acc[(s * rows + idx) * head_dim + d] * __expf(m[s * rows + idx] - mx);
        out[(size_t)row * out_stride_m + (size_t)head * out_stride_h + d] = __float2half_rn(a * inv);
    }
}

template <int D, int STAGES>
mf_status launch_pf(MfContext *ctx, const CUtensorMap &tm_k, const CUtensorMap &tm_v, const PrefillParams &p, dim3 grid)
{
    constexpr uint32_t kDyn = STAGES * 2 * kTileKeys * D * 2 + 2 * STAGES * 8 + 16 + 1024;
    static bool configured[64] = {};
    auto kern = prefill_kernel<D, STAGES>;
    if (ctx->device < 64 && !configured[ctx->device]) {
        mf_status st = check_cuda(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kDyn),
                                  "cudaFuncSetAttribute(prefill)");
        if (st != MF_OK) return st;
        configured[ctx->device] = true;
    }
    kern<<<grid, kPfThreads, kDyn, ctx->stream>>>(tm_k, tm_v, p);
    return check_launch(ctx, "prefill_kernel");
}

}  // namespace

mf_status launch_prefill_tc(MfContext *ctx, const void *q, const void *k, const void *v, void *out,
                            const SdpaPrefillSplitKParams &sp, bool *handled, const MfPagedKv *paged, uint32_t seq);

mf_status launch_prefill(MfContext *ctx, const void *q, const void *k, const void *v, void *out,
                         const SdpaPrefillSplitKParams &sp, const MfPagedKv *paged, uint32_t seq)
{
    const SdpaPrefillParams &b = sp.base;
    const uint32_t D = b.head_dim;
    if (D != 64 && D != 128)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "Prefill only supports head_dim=64 or 128, got %u", D);
    if (b.stride_k_s != D || b.stride_v_s != D)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "Prefill: K/V row stride must equal head_dim");
    if (b.q_len == 0 || b.kv_len == 0 || sp.n_heads == 0) return MF_OK;
    if (b.group_size == 0 || sp.n_heads % b.group_size != 0)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "Prefill: n_heads %u / group_size %u", sp.n_heads, b.group_size);
    if (paged) {
        const uint32_t P = paged->page_size;
        if (P < 8 || (P & (P - 1)) != 0)
            return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "Paged prefill: page size %u (power of two >= 8)", P);
        if (seq >= paged->batch) return fail(ctx, MF_ERR_INVALID_OPERATION, "Paged prefill: sequence %u of %u", seq, paged->batch);
        if (((uint64_t)b.kv_len + P - 1) / P > paged->page_table_stride)
            return fail(ctx, MF_ERR_INVALID_OPERATION, "Paged prefill: kv_len %u exceeds the page table", b.kv_len);
        if (paged->head_dim != D || sp.n_heads / b.group_size != paged->n_kv_heads)
            return fail(ctx, MF_ERR_INVALID_SHAPE, "Paged prefill: cache is %u kv heads x %u, call has %u x %u", paged->n_kv_heads,
                        paged->head_dim, sp.n_heads / b.group_size, D);
    } else {
        if (b.k_stride_h % D || b.v_stride_h % D)
            return fail(ctx, MF_ERR_INVALID_SHAPE, "Prefill: K/V head strides must be multiples of head_dim");
        if ((uint64_t)b.kv_len * D > b.k_stride_h || (uint64_t)b.kv_len * D > b.v_stride_h)
            return fail(ctx, MF_ERR_INVALID_OPERATION, "Prefill: kv_len %u exceeds the cache capacity", b.kv_len);
    }
    if ((b.q_stride_h | b.q_stride_m) & 1u || (b.out_stride_h | b.out_stride_m) & 1u ||
        (reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out)) & 3u)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "Prefill: q/output strides must be even and pointers 4-byte aligned");
    if (ctx->prefill_impl != 1) {
        // tcgen05 / TMEM kernel: unsplit, chunks of 64 rows or more, contiguous cache or pages of 8-128 rows
        bool handled = false;
        mf_status st_tc = launch_prefill_tc(ctx, q, k, v, out, sp, &handled, paged, seq);
        if (st_tc != MF_OK || handled) return st_tc;
        if (ctx->prefill_impl == 2)
            return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "Prefill: shape outside the tcgen05 kernel's envelope");
    }
    const uint32_t cache_heads = sp.n_heads / b.group_size;
    const uint32_t q_tiles = (b.q_len + kPfTileM - 1) / kPfTileM;
    uint32_t split_k = std::max(1u, sp.split_k);
    // Split ranges follow splitk_tile_range (flash_prefill.metal:452-457): 32-key tiles.
    const uint32_t tiles32 = (b.kv_len + 31) / 32;
    split_k = std::min(split_k, std::max(1u, tiles32));
    const uint32_t keys_per_split = ((tiles32 + split_k - 1) / split_k) * 32;

    PrefillParams p{};
    p.q = static_cast<const __half *>(q);
    p.out = static_cast<__half *>(out);
    p.status = ctx->d_status;
    p.q_len = b.q_len;
    p.kv_len = b.kv_len;
    p.query_offset = b.query_offset;
    p.group = b.group_size;
    p.q_stride_h = b.q_stride_h;
    p.q_stride_m = b.q_stride_m;
    p.out_stride_h = b.out_stride_h;
    p.out_stride_m = b.out_stride_m;
    p.k_rows_h = b.k_stride_h / D;
    p.v_rows_h = b.v_stride_h / D;
    p.n_heads = sp.n_heads;
    p.split_k = split_k;
    p.keys_per_split = split_k > 1 ? keys_per_split : b.kv_len;
    p.scale_log2 = b.scale * 1.4426950408889634f;
    mf_status st;
    if (split_k > 1) {
        const uint64_t rows = (uint64_t)split_k * sp.n_heads * b.q_len;
        const uint64_t need = kCounterRegionBytes + rows * (D + 2) * 4;
        if ((st = ensure_scratch(ctx, need)) != MF_OK) return st;
        float *base = reinterpret_cast<float *>(static_cast<char *>(ctx->scratch) + kCounterRegionBytes);
        p.part_acc = base;
        p.part_m = base + rows * D;
        p.part_l = p.part_m + rows;
    }
    CUtensorMap tm_k, tm_v;
    if (paged) {
        p.page_table_row = paged->page_table + (size_t)seq * paged->page_table_stride;
        p.page_size = paged->page_size;
        p.n_kv_heads = paged->n_kv_heads;
        const uint64_t rows = (uint64_t)paged->n_pages * paged->n_kv_heads * paged->page_size;
        const uint32_t box_rows = std::min(paged->page_size, kTileKeys);
        if ((st = get_tensor_map(ctx, paged->k_pool, rows, D, box_rows, 64, &tm_k)) != MF_OK) return st;
        if ((st = get_tensor_map(ctx, paged->v_pool, rows, D, box_rows, 64, &tm_v)) != MF_OK) return st;
    } else {
        if ((st = get_tensor_map(ctx, k, (uint64_t)cache_heads * p.k_rows_h, D, kTileKeys, 64, &tm_k)) != MF_OK) return st;
        if ((st = get_tensor_map(ctx, v, (uint64_t)cache_heads * p.v_rows_h, D, kTileKeys, 64, &tm_v)) != MF_OK) return st;
    }
    dim3 grid(q_tiles, sp.n_heads, split_k);
    st = (D == 128) ? launch_pf<128, 4>(ctx, tm_k, tm_v, p, grid) : launch_pf<64, 4>(ctx, tm_k, tm_v, p, grid);
    if (st != MF_OK || split_k == 1) return st;
    prefill_reduce_kernel<<<dim3(b.q_len, sp.n_heads), 128, 0, ctx->stream>>>(
        p.part_acc, p.part_m, p.part_l, split_k, sp.n_heads, b.q_len, D, p.out, b.out_stride_h, b.out_stride_m);
    return check_launch(ctx, "prefill_reduce_kernel");
}

}  // namespace mf
