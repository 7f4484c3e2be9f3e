// GQA flash-decode over a contiguous or paged F16 KV cache for sm_100a, with the
// append of the step's new token and the RoPE of q fused in.
//
// Replaces flash_decode_warp_tiled_m1_half2/half4 (flash_decode.metal:146-490),
// run_flash_head_layout_stage (:107-144) and, when rope/append are set, RopeStage
// (rope_common.metal:27-63) and the K/V part of kv_prep_fused_kernel_f16
// (kv_prep_fused.metal:89-122).  The arithmetic contract kept from those kernels:
// q and the appended k are rounded to f16 after RoPE, scores are f16 x f16
// products accumulated in f32 and multiplied by `scale`, the running max starts
// at -1e30, non-finite scores count as -1e30, accumulation is f32, and the result
// is acc/l (acc when |l| <= 1e-6), non-finite -> 0, one rounding to f16.
//
// Shape of the kernel (not the reference's): the reference runs one threadgroup
// per query head and walks all keys serially, so K/V are read once per QUERY
// head.  Here one CTA processes spans of 64-key tiles of one (sequence, kv head)
// unit for all G query heads of the group at once, so K/V cross HBM once per KV
// head.  A producer warp streams K/V tiles into a multi-stage shared-memory ring
// with TMA tensor loads (one box per page and 64-column half, 128-byte swizzle)
// signalled through mbarriers; four consumer warps take 16 keys each, compute
// S^T = K Q^T and O^T += V^T P^T on mma.sync m16n8k16 (keys / dims on the M side,
// the query group on the 8-wide N side), keep online-softmax state in registers
// (row max by warp shuffles) and combine at the end of the span.  Spans that do
// not cover a whole unit write unnormalised f32 partials; the CTA that finishes a
// unit last (an atomic ticket, no waiting) merges them with the log-sum-exp rule
// of flash_prefill.metal:843-888.
#include <algorithm>

#include "internal.hpp"
#include "ptx.cuh"
#include "push.cuh"

namespace mf {

namespace {

constexpr uint32_t kConsumerWarps = 4;
constexpr uint32_t kConsumerThreads = kConsumerWarps * 32;
constexpr uint32_t kThreads = kConsumerThreads + 32;
constexpr float kNegSentinel = -1e30f;
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s per barrier wait
constexpr float kLn2 = 0.6931471805599453f;
constexpr uint32_t kMergeFlight = 20;  // partials whose loads are in flight together in the merge
constexpr uint32_t kMergeFlightFew = 8;                // ... for units cut in at most this many parts


template <int D, int NT, int STAGES, bool CL = false>
struct Smem {
    static constexpr uint32_t kHP = 8 * NT;                    // padded heads per group
    static constexpr uint32_t kTileBytes = kTileKeys * D * 2;  // one K or V tile
    static constexpr uint32_t kStageBytes = 2 * kTileBytes;
    static constexpr uint32_t kCombStride = D / 2 + 4;       // floats per head row (half of D per pass)
    static constexpr uint32_t kQStride = D + 8;              // halves per head row
    static constexpr uint32_t kOffComb = STAGES * kStageBytes;
    static constexpr uint32_t kCombBytes = kConsumerWarps * kHP * kCombStride * 4;
    static constexpr uint32_t kOffQ = kOffComb + kCombBytes;
    static constexpr uint32_t kQBytes = kHP * kQStride * 2;
    static constexpr uint32_t kOffMl = kOffQ + kQBytes;
    static constexpr uint32_t kMlBytes = kConsumerWarps * kHP * 2 * 4;
    static constexpr uint32_t kOffMerge = kOffMl + kMlBytes;
    static constexpr uint32_t kMergeBytes = kHP * 2 * 4;
    // Cluster form: what the other CTAs of the cluster store here for this CTA to reduce.  [source CTA][the
    // D / C dims this CTA owns][HP heads] accumulators (D * HP floats whatever the cluster size C) and
    // [source CTA (up to 16)][HP] (m, l) pairs.  Dedicated: a fast CTA stores while a slow one still streams tiles.
    static constexpr uint32_t kOffRecv = kOffMerge + kMergeBytes;
    static constexpr uint32_t kRecvAccBytes = kHP * D * 4;
    static constexpr uint32_t kRecvBytes = CL ? kRecvAccBytes + 16 * kHP * 2 * 4 : 0;  // only the cluster form has it
    static constexpr uint32_t kOffBar = kOffRecv + kRecvBytes;
    static constexpr uint32_t kBarBytes = 2 * STAGES * 8;
    static constexpr uint32_t kOffFlags = kOffBar + kBarBytes;
    static constexpr uint32_t kTotal = kOffFlags + 16;
    static constexpr uint32_t kDynamic = kTotal + 1024;  // slack for 1024-byte alignment
};

// Iterates the work items of one CTA, from the explicit plan or, for uniform
// lengths, computed from the CTA index.
__device__ __forceinline__ uint32_t kv_len_of(const DecodeParams &p, uint32_t seq)
{
    return p.kv_lens ? p.kv_lens[seq] : p.uniform_kv_len;
}

template <bool CL>
struct ItemCursor {
    const DecodeParams &p;
    uint32_t idx, end;       // explicit mode
    uint32_t flat, flat_end; // uniform mode
    bool cluster_pending;    // cluster form: the one item of this CTA's cluster has not been handed out yet
    uint32_t len;            // kv length of the item next() handed out last
    // explicit mode: the item after the current one and its length, fetched while the current item's tiles stream
    // (two dependent loads less between the last tile of one item and the first of the next)
    WorkItem ahead;
    uint32_t ahead_len;
    __device__ void fetch_ahead()
    {
        if (idx < end) {
            ahead = p.items[idx];
            ahead_len = kv_len_of(p, ahead.seq);
        }
    }
    __device__ ItemCursor(const DecodeParams &pp, uint32_t cta) : p(pp)
    {
        cluster_pending = CL;
        len = ahead_len = 0;
        ahead = WorkItem{};
        if (CL) {
            idx = end = flat = flat_end = 0;
        } else if (p.items) {
            idx = p.cta_item_begin[cta];
            end = p.cta_item_begin[cta + 1];
            flat = flat_end = 0;
            fetch_ahead();
        } else {
            idx = end = 0;
            flat = cta * p.uniform_span;
            flat_end = min(p.uniform_total, flat + p.uniform_span);
        }
    }
    __device__ bool next(WorkItem &it)
    {
        if (CL) {
            // One item per cluster; this CTA takes an equal share of its tiles (the first `rem` CTAs one more).
            if (!cluster_pending) return false;
            cluster_pending = false;
            const uint32_t C = p.cluster_size, c = blockIdx.x / C, r = cluster_cta_rank();
            if (p.items) {
                it = p.items[c];
            } else {
                const uint32_t u = c / p.uniform_parts, part = c - u * p.uniform_parts;
                it.seq = u / p.n_kv_heads;
                it.kvh = u - it.seq * p.n_kv_heads;
                it.tile_begin = part * p.uniform_span;
                it.tile_end = min(p.uniform_tiles, it.tile_begin + p.uniform_span);
                it.unit = u;
                it.n_parts = p.uniform_parts;
                it.first_slot = u * p.uniform_parts;
                it.slot = it.first_slot + part;
            }
            const uint32_t tiles = it.tile_end - it.tile_begin, base = tiles / C, rem = tiles - base * C;
            it.tile_begin += r * base + min(r, rem);
            it.tile_end = it.tile_begin + base + (r < rem ? 1u : 0u);
            len = kv_len_of(p, it.seq);
            return true;
        }
        if (p.items) {
            if (idx >= end) return false;
            it = ahead;
            len = ahead_len;
            ++idx;
            fetch_ahead();
            return true;
        }
        if (flat >= flat_end) return false;
        const uint32_t T = p.uniform_tiles;
        if (p.uniform_parts) {
            // flat / span is the CTA index: unit = cta / parts, range `cta % parts` of the unit
            const uint32_t cta = flat / p.uniform_span;
            const uint32_t u = cta / p.uniform_parts, part = cta - u * p.uniform_parts;
            it.seq = u / p.n_kv_heads;
            it.kvh = u - it.seq * p.n_kv_heads;
            it.tile_begin = part * p.uniform_span;
            it.tile_end = min(T, it.tile_begin + p.uniform_span);
            it.unit = u;
            it.n_parts = p.uniform_parts;
            it.first_slot = u * p.uniform_parts;
            it.slot = it.first_slot + part;
            flat = flat_end;
            len = kv_len_of(p, it.seq);
            return true;
        }
        const uint32_t u = flat / T;
        const uint32_t tb = flat - u * T;
        const uint32_t te = min(T, tb + (flat_end - flat));
        const uint32_t c_first = (u * T) / p.uniform_span;
        const uint32_t c_last = ((u + 1) * T - 1) / p.uniform_span;
        it.seq = u / p.n_kv_heads;
        it.kvh = u - it.seq * p.n_kv_heads;
        it.tile_begin = tb;
        it.tile_end = te;
        it.unit = u;
        it.n_parts = c_last - c_first + 1;
        it.first_slot = u + c_first;
        it.slot = u + flat / p.uniform_span;
        flat += te - tb;
        len = kv_len_of(p, it.seq);
        return true;
    }
};

// Byte offset of (row, 16-byte chunk `c16` of the D*2-byte row) inside a K or V tile.
// A tile is a sequence of TMA boxes of 2^rpb_log2 rows (one page, or 64 rows); each box
// is laid out [64-column half][rows][128 B] with the TMA 128-byte swizzle.
template <int D>
__device__ __forceinline__ uint32_t tile_off(uint32_t row, uint32_t c16, uint32_t rpb_log2)
{
    constexpr uint32_t kRowLog2 = (D == 128) ? 8 : 7;
    const uint32_t box = row >> rpb_log2;
    const uint32_t rr = row & ((1u << rpb_log2) - 1u);
    return (box << (rpb_log2 + kRowLog2)) + ((c16 >> 3) << (rpb_log2 + 7)) + (rr << 7) +
           (((c16 & 7) ^ (row & 7)) << 4);
}

// One RoPE'd element pair, rounded to f16 exactly as kv_prep_fused.metal:74-82.
__device__ __forceinline__ void rope_pair(float xi, float xj, float c, float s, __half &oi,
                                          __half &oj)
{
    oi = __float2half_rn(__fsub_rn(__fmul_rn(xi, c), __fmul_rn(xj, s)));
    oj = __float2half_rn(__fadd_rn(__fmul_rn(xj, c), __fmul_rn(xi, s)));
}

using push::push_signal_and_merge;
using push::push_store;
using push::push_wait_for_mergers;

template <int D, int NT, int STAGES, int MINB, bool CL = false>
__global__ void __launch_bounds__(kThreads, MINB)
decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
              const DecodeParams p)
{
    using S = Smem<D, NT, STAGES, CL>;
    constexpr uint32_t HP = S::kHP;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t tid = threadIdx.x;
    const uint32_t warp = tid >> 5;
    const uint32_t lane = tid & 31;
    const uint32_t bar_full = smem_base + S::kOffBar;
    const uint32_t bar_empty = bar_full + STAGES * 8;
    volatile uint32_t *flags = reinterpret_cast<volatile uint32_t *>(smem + S::kOffFlags);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, kConsumerWarps);
        }
        flags[0] = 0;  // abort
        flags[1] = 0;  // merge ticket broadcast
        mbar_fence_init();
        fence_proxy_async();
    }
    __syncthreads();

    const uint32_t rows_per_box = p.page_table ? min(p.page_size, kTileKeys) : kTileKeys;
    const uint32_t boxes_per_tile = kTileKeys / rows_per_box;
    const uint32_t rpb_log2 = 31 - __clz(rows_per_box);

    // Relaxed launches let the next launch of the stream be scheduled right away (it sets up, and its
    // producer may stream its own K/V, while this grid works); strict ones do so only after their wait.
    // Cluster-form launches release theirs when their own last tile has been requested: the next launch then
    // fills its ring while this one combines and writes, not while it still streams (its requests would queue in
    // front of tiles this launch is waiting for).
    if (!p.strict_release && !p.release_late) grid_launch_dependents();
    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------ producer ---
        if (lane == 0) {
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_v);
        }
        // K/V pages of earlier tokens were written at least one launch ago; only when the caller
        // appended with a separate kernel right before must the stream of tiles wait for it.
        if (!p.early_stream) grid_dependency_wait();
        const uint64_t policy = l2_policy_evict_first();
        ItemCursor<CL> cur(p, blockIdx.x);
        WorkItem it;
        uint32_t stage = 0, phase = 0, issued = 0;
        while (cur.next(it)) {
            const uint32_t L = cur.len;
            // Paged: the ids of 32 pages travel one per lane, a chunk ahead of the tiles that use them (a lookup
            // per tile, even issued one tile early, put a global-load latency into every tile of the stream).
            const bool paged = p.page_table != nullptr;
            const uint32_t *pt_row = paged ? p.page_table + (size_t)it.seq * p.pt_stride : nullptr;
            const uint32_t n_pg = paged ? min((L + p.page_size - 1) / p.page_size, p.pt_stride) : 0u;
            uint32_t chunk = paged ? (it.tile_begin * kTileKeys) / p.page_size : 0u;
            auto load_ids = [&](uint32_t base) -> uint32_t { return base + lane < n_pg ? __ldg(pt_row + base + lane) : 0u; };
            uint32_t ids = load_ids(chunk), ids_next = load_ids(chunk + 32);
            for (uint32_t t = it.tile_begin; t < it.tile_end; ++t) {
                // Row of this lane's box inside the K / V tensor.
                const uint32_t tok = t * kTileKeys + lane * rows_per_box;
                bool valid = lane < boxes_per_tile;
                int32_t rk, rv;
                if (paged) {
                    if ((t * kTileKeys) / p.page_size >= chunk + 32) {
                        ids = ids_next;
                        chunk += 32;
                        ids_next = load_ids(chunk + 32);
                    }
                    const uint32_t pg = tok / p.page_size;
                    const uint32_t page = __shfl_sync(0xffffffffu, ids, (pg - chunk) & 31u);
                    // rows past the sequence, or past the page table when the device-side length is larger
                    // than the table allows (the consumers report that), are not fetched
                    valid = valid && tok < L && pg < p.pt_stride;
                    rk = rv = static_cast<int32_t>((page * p.n_kv_heads + it.kvh) * p.page_size + tok % p.page_size);
                } else {
                    rk = static_cast<int32_t>(it.seq * p.k_rows_b + it.kvh * p.k_rows_h + tok);
                    rv = static_cast<int32_t>(it.seq * p.v_rows_b + it.kvh * p.v_rows_h + tok);
                }
                if (!flags[0] && !mbar_wait_bounded(bar_empty + stage * 8, phase ^ 1, kWaitLimitNs)) {
                    flags[0] = 1;
                    atomicOr(p.status, 1u);
                }
                const uint32_t n_valid = __popc(__ballot_sync(0xffffffffu, valid));
                const uint32_t full = bar_full + stage * 8;
                if (lane == 0) mbar_arrive_expect_tx(full, n_valid * rows_per_box * D * 4);
                __syncwarp();
                if (valid) {
                    const uint32_t dst_k = smem_base + stage * S::kStageBytes + lane * rows_per_box * (D * 2);
                    const uint32_t dst_v = dst_k + S::kTileBytes;
                    if (D == 128 && p.whole_rows) {
                        // one copy per page and tensor: both 64-column halves of every row
                        tma_load_3d_hint(dst_k, &tm_k, 0, rk, 0, full, policy);
                        tma_load_3d_hint(dst_v, &tm_v, 0, rv, 0, full, policy);
                    } else {
#pragma unroll
                        for (int h = 0; h < D / 64; ++h) {
                            tma_load_2d_hint(dst_k + h * rows_per_box * 128, &tm_k, h * 64, rk, full, policy);
                            tma_load_2d_hint(dst_v + h * rows_per_box * 128, &tm_v, h * 64, rv, full, policy);
                        }
                    }
                }
                ++issued;
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
        if (p.release_late) grid_launch_dependents();
        // After an abort the consumers no longer wait for the ring: make sure our
        // own copies have landed before the CTA gives its shared memory back.
        if (flags[0]) {
            const uint32_t n = issued < (uint32_t)STAGES ? issued : (uint32_t)STAGES;
            for (uint32_t i = 0; i < n; ++i) {
                const uint32_t s = (stage + STAGES - 1 - i) % STAGES;
                const uint32_t ph = (s < stage) ? phase : (phase ^ 1);
                (void)mbar_wait_bounded(bar_full + s * 8, ph, kWaitLimitNs);
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumers ---
    // q, the new k/v, the partial slots and tickets may all have been written by the previous launch.
    grid_dependency_wait();
    // A strict launch releases its dependents only here: the launch behind it then cannot start before
    // every CTA of this one has seen the launch in front complete, which is what bounds the set of launches
    // an early K/V stream can race with.
    if (p.strict_release) grid_launch_dependents();
    if (p.push_wait_mask) push_wait_for_mergers(p, tid);
    float *comb = reinterpret_cast<float *>(smem + S::kOffComb);
    __half *q_s = reinterpret_cast<__half *>(smem + S::kOffQ);
    float *ml_s = reinterpret_cast<float *>(smem + S::kOffMl);
    float *merge_s = reinterpret_cast<float *>(smem + S::kOffMerge);
    const uint32_t G = p.group;
    const uint32_t half_d = D / 2;

    ItemCursor<CL> cur(p, blockIdx.x);
    WorkItem it;
    uint32_t stage = 0, phase = 0;
    while (cur.next(it)) {
        const uint32_t L = cur.len;
        const uint32_t n_tiles = (L + kTileKeys - 1) / kTileKeys;
        const uint32_t pos = p.rope_positions ? p.rope_positions[it.seq]
                                              : (p.kv_lens ? (L ? L - 1 : 0) : p.rope_position);
        const __half *cos_row = p.cos_t + (size_t)pos * half_d;
        const __half *sin_row = p.sin_t + (size_t)pos * half_d;

        // ---- q (optionally roped, rounded to f16) -> shared memory -----------------
        // Every global load of this prologue is issued before the first one is used: q of the group's heads, the
        // position's cos / sin pair, and - in the CTA that will meet the sequence's last tile - the new k and v row
        // and the id of the page they go to.  One memory latency instead of one per pass and one more at the last tile.
        named_bar_sync(1, kConsumerThreads);  // previous item is done with q_s / comb
        constexpr uint32_t kQPasses = (HP * (D / 2)) / kConsumerThreads;
        static_assert((HP * (D / 2)) % kConsumerThreads == 0 && kConsumerThreads % (D / 2) == 0, "q staging");
        const uint32_t pr = tid % half_d;  // the same pair of dims in every pass
        const uint32_t di = p.rope_mode == MF_ROPE_MODE_NORMAL ? 2 * pr : pr;
        const uint32_t dj = p.rope_mode == MF_ROPE_MODE_NORMAL ? di + 1 : pr + half_d;
        __half qi[kQPasses], qj[kQPasses];
#pragma unroll
        for (uint32_t j = 0; j < kQPasses; ++j) {
            const uint32_t g = (tid + j * kConsumerThreads) / half_d;
            qi[j] = qj[j] = __float2half_rn(0.f);
            if (g < G) {
                const __half *src = p.q + (size_t)it.seq * p.q_stride_b + (size_t)(it.kvh * G + g) * p.q_stride_h;
                qi[j] = src[di];
                qj[j] = src[dj];
            }
        }
        float cs = 1.f, sn = 0.f;
        if (p.rope) {
            cs = __half2float(cos_row[pr]);
            sn = __half2float(sin_row[pr]);
        }
        // the row this step appends, if this CTA's span ends the sequence
        const bool ends_seq = p.append && it.tile_begin < n_tiles && it.tile_end >= n_tiles;
        __half kn_i = __float2half_rn(0.f), kn_j = kn_i, vn = kn_i;
        uint32_t new_page = 0;
        bool store_ok = true;
        if (ends_seq) {
            if (tid < half_d) {
                const __half *ks = p.k_new + (size_t)it.seq * p.knew_stride_b + (size_t)it.kvh * D;
                kn_i = ks[di];
                kn_j = ks[dj];
            }
            if (tid < (uint32_t)D) vn = p.v_new[(size_t)it.seq * p.knew_stride_b + (size_t)it.kvh * D + tid];
            if (p.page_table) {
                // The page id of the new row comes from the caller's device-side table: one that is not a page
                // of this pool (or a length the table has no entry for) skips the store and the splice and
                // raises the status bit; the output of that sequence is then not meaningful.
                store_ok = (L - 1) / p.page_size < p.pt_stride;
                if (store_ok) {
                    new_page = p.page_table[(size_t)it.seq * p.pt_stride + (L - 1) / p.page_size];
                    store_ok = new_page < p.n_pages;
                }
            }
        }
#pragma unroll
        for (uint32_t j = 0; j < kQPasses; ++j) {
            const uint32_t g = (tid + j * kConsumerThreads) / half_d;
            __half oi = qi[j], oj = qj[j];
            if (g < G) {
                if (p.rope) rope_pair(__half2float(oi), __half2float(oj), cs, sn, oi, oj);
                if (p.q_rot && it.tile_begin == 0) {
                    __half *dst = p.q_rot + (size_t)it.seq * p.q_stride_b + (size_t)(it.kvh * G + g) * p.q_stride_h;
                    dst[di] = oi;
                    dst[dj] = oj;
                }
            }
            q_s[g * S::kQStride + di] = oi;
            q_s[g * S::kQStride + dj] = oj;
        }
        if (ends_seq && p.rope) rope_pair(__half2float(kn_i), __half2float(kn_j), cs, sn, kn_i, kn_j);
        named_bar_sync(1, kConsumerThreads);

        // B fragments of Q^T: [k = 16 dims][n = 8 heads] per k-step and n-tile.
        uint32_t bq[NT][D / 16][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const __half *row = q_s + (nt * 8 + (lane >> 2)) * S::kQStride + 2 * (lane & 3);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                bq[nt][ks][0] = *reinterpret_cast<const uint32_t *>(row + ks * 16);
                bq[nt][ks][1] = *reinterpret_cast<const uint32_t *>(row + ks * 16 + 8);
            }
        }

        float m_run[NT][2], l_run[NT][2];
        float o[NT][D / 16][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            m_run[nt][0] = m_run[nt][1] = kNegSentinel;
            l_run[nt][0] = l_run[nt][1] = 0.f;
#pragma unroll
            for (int mt = 0; mt < D / 16; ++mt) o[nt][mt][0] = o[nt][mt][1] = o[nt][mt][2] = o[nt][mt][3] = 0.f;
        }

        for (uint32_t t = it.tile_begin; t < it.tile_end; ++t) {
            if (!flags[0] && !mbar_wait_bounded(bar_full + stage * 8, phase, kWaitLimitNs)) {
                flags[0] = 1;
                atomicOr(p.status, 2u);
            }
            uint8_t *k_tile = smem + stage * S::kStageBytes;
            uint8_t *v_tile = k_tile + S::kTileBytes;
            const uint32_t k_addr = smem_base + stage * S::kStageBytes;
            const uint32_t v_addr = k_addr + S::kTileBytes;
            const uint32_t key0 = t * kTileKeys;
            const bool last_tile = (t + 1 == n_tiles);

            if (last_tile) {
                // The tile that holds position L-1: splice in the token appended by
                // this step (and store it to the cache), then clear V rows past L so
                // that stale or never-written rows cannot leak NaNs through 0 * NaN.
                const uint32_t r_new = (L - 1) - key0;
                if (p.append && !store_ok && tid == 0) atomicOr(p.status, kStatusBadPage);
                if (p.append && store_ok) {
                    size_t krow, vrow;
                    if (p.page_table) {
                        krow = vrow = ((size_t)new_page * p.n_kv_heads + it.kvh) * p.page_size + (L - 1) % p.page_size;
                    } else {
                        krow = (size_t)it.seq * p.k_rows_b + (size_t)it.kvh * p.k_rows_h + (L - 1);
                        vrow = (size_t)it.seq * p.v_rows_b + (size_t)it.kvh * p.v_rows_h + (L - 1);
                    }
                    if (tid < half_d) {  // the pair this thread roped in the prologue
                        p.k_base[krow * D + di] = kn_i;
                        p.k_base[krow * D + dj] = kn_j;
                        *reinterpret_cast<__half *>(k_tile + tile_off<D>(r_new, di >> 3, rpb_log2) + (di & 7) * 2) = kn_i;
                        *reinterpret_cast<__half *>(k_tile + tile_off<D>(r_new, dj >> 3, rpb_log2) + (dj & 7) * 2) = kn_j;
                    }
                    if (tid < (uint32_t)D) {
                        p.v_base[vrow * D + tid] = vn;
                        *reinterpret_cast<__half *>(v_tile + tile_off<D>(r_new, tid >> 3, rpb_log2) + (tid & 7) * 2) = vn;
                    }
                }
                const uint32_t first_dead = L - key0;  // 1..64
                const uint32_t n_chunks = (kTileKeys - first_dead) * (D / 8);
                for (uint32_t c = tid; c < n_chunks; c += kConsumerThreads) {
                    const uint32_t row = first_dead + c / (D / 8);
                    const uint32_t c16 = c % (D / 8);
                    *reinterpret_cast<uint4 *>(v_tile + tile_off<D>(row, c16, rpb_log2)) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async();  // order these writes before the ring's next TMA refill
                named_bar_sync(2, kConsumerThreads);
            }

            const uint32_t wkey0 = key0 + warp * 16;
            if (wkey0 < L) {
                // ---- S^T (16 keys x 8*NT heads) = K_tile Q^T ---------------------------
                // two accumulators per n-tile (even and odd k-steps): the products of a tile form two dependent
                // chains of D / 32 instead of one of D / 16
                float c[NT][4], c_odd[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.f;
                    c_odd[nt][0] = c_odd[nt][1] = c_odd[nt][2] = c_odd[nt][3] = 0.f;
                }
                {
                    const uint32_t row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks) {
                        uint32_t a[4];
                        ldmatrix_x4(a, k_addr + tile_off<D>(row, 2 * ks + (lane >> 4), rpb_log2));
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) mma_m16n8k16((ks & 1) ? c_odd[nt] : c[nt], a, bq[nt][ks][0], bq[nt][ks][1]);
                    }
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    c[nt][0] += c_odd[nt][0];
                    c[nt][1] += c_odd[nt][1];
                    c[nt][2] += c_odd[nt][2];
                    c[nt][3] += c_odd[nt][3];
                }
                // ---- online softmax over this warp's 16 keys ---------------------------
                const uint32_t kr0 = wkey0 + (lane >> 2);
                const bool dead0 = kr0 >= L, dead1 = kr0 + 8 >= L;
                uint32_t bp[NT][2];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    float s0 = c[nt][0] * p.scale_log2, s1 = c[nt][1] * p.scale_log2;
                    float s2 = c[nt][2] * p.scale_log2, s3 = c[nt][3] * p.scale_log2;
                    if (dead0 || !(fabsf(s0) <= 3.0e38f)) s0 = kNegSentinel;
                    if (dead0 || !(fabsf(s1) <= 3.0e38f)) s1 = kNegSentinel;
                    if (dead1 || !(fabsf(s2) <= 3.0e38f)) s2 = kNegSentinel;
                    if (dead1 || !(fabsf(s3) <= 3.0e38f)) s3 = kNegSentinel;
                    float mx0 = fmaxf(s0, s2), mx1 = fmaxf(s1, s3);
#pragma unroll
                    for (int off = 4; off <= 16; off <<= 1) {
                        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
                        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
                    }
                    const float mn0 = fmaxf(m_run[nt][0], mx0), mn1 = fmaxf(m_run[nt][1], mx1);
                    const float a0 = fast_exp2(m_run[nt][0] - mn0), a1 = fast_exp2(m_run[nt][1] - mn1);
                    m_run[nt][0] = mn0;
                    m_run[nt][1] = mn1;
                    // Masked keys get weight 0 even when the whole row so far is masked
                    // (then s - m would be 0, not -inf).
                    const float p0 = dead0 ? 0.f : fast_exp2(s0 - mn0);
                    const float p1 = dead0 ? 0.f : fast_exp2(s1 - mn1);
                    const float p2 = dead1 ? 0.f : fast_exp2(s2 - mn0);
                    const float p3 = dead1 ? 0.f : fast_exp2(s3 - mn1);
                    l_run[nt][0] = l_run[nt][0] * a0 + (p0 + p2);
                    l_run[nt][1] = l_run[nt][1] * a1 + (p1 + p3);
#pragma unroll
                    for (int mt = 0; mt < D / 16; ++mt) {
                        o[nt][mt][0] *= a0;
                        o[nt][mt][1] *= a1;
                        o[nt][mt][2] *= a0;
                        o[nt][mt][3] *= a1;
                    }
                    bp[nt][0] = movmatrix_trans(pack_f16x2(p0, p1));
                    bp[nt][1] = movmatrix_trans(pack_f16x2(p2, p3));
                }
                // ---- O^T (D dims x heads) += V_tile^T P^T ------------------------------
                {
                    const uint32_t row = warp * 16 + (lane & 7) + (lane >> 4) * 8;
#pragma unroll
                    for (int mt = 0; mt < D / 16; ++mt) {
                        uint32_t a[4];
                        ldmatrix_x4_trans(a, v_addr + tile_off<D>(row, 2 * mt + ((lane >> 3) & 1), rpb_log2));
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) mma_m16n8k16(o[nt][mt], a, bp[nt][0], bp[nt][1]);
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

        // ---- combine the four warps' states ------------------------------------------
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int off = 4; off <= 16; off <<= 1) {
                l_run[nt][0] += __shfl_xor_sync(0xffffffffu, l_run[nt][0], off);
                l_run[nt][1] += __shfl_xor_sync(0xffffffffu, l_run[nt][1], off);
            }
            if (lane < 4) {
                float *dst = ml_s + ((warp * HP) + nt * 8 + 2 * lane) * 2;
                dst[0] = m_run[nt][0];
                dst[1] = l_run[nt][0];
                dst[2] = m_run[nt][1];
                dst[3] = l_run[nt][1];
            }
        }
        named_bar_sync(1, kConsumerThreads);
        float fac[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint32_t h0 = nt * 8 + 2 * (lane & 3);
            float ma0 = kNegSentinel, ma1 = kNegSentinel;
#pragma unroll
            for (uint32_t w = 0; w < kConsumerWarps; ++w) {
                ma0 = fmaxf(ma0, ml_s[(w * HP + h0) * 2]);
                ma1 = fmaxf(ma1, ml_s[(w * HP + h0 + 1) * 2]);
            }
            fac[nt][0] = fast_exp2(m_run[nt][0] - ma0);
            fac[nt][1] = fast_exp2(m_run[nt][1] - ma1);
        }

        const bool direct = (it.n_parts == 1);
        const bool partial_out = (p.out_acc != nullptr);
        // Cluster form: CTA r of the cluster owns the dims [r * D / C, (r + 1) * D / C) of every head.  Each CTA
        // stores its combined accumulators straight into the owners' shared memory (and its (m, l) pairs into
        // everybody's), m in the scaled log2 domain; after one cluster barrier every owner reduces locally.
        constexpr bool cl = CL;  // a separate instantiation: the plain form carries none of this
        const uint32_t C = cl ? p.cluster_size : 1u, crank = cl ? cluster_cta_rank() : 0u;
        const uint32_t own_dims = D / C;  // C is a power of two up to 16
        const uint32_t recv_acc_addr = smem_base + S::kOffRecv, recv_ml_addr = recv_acc_addr + S::kRecvAccBytes;
        if (cl) {
            // One item per CTA in this form, so the ring is idle by now: its first bytes take the four warps'
            // accumulators at full width, in one pass.
            constexpr uint32_t kFS = D + 4;  // floats per head row
            float *cf = reinterpret_cast<float *>(smem);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint32_t h0 = nt * 8 + 2 * (lane & 3);
                float *c0 = cf + (warp * HP + h0) * kFS;
                float *c1 = c0 + kFS;
#pragma unroll
                for (int mt = 0; mt < D / 16; ++mt) {
                    const uint32_t d0 = mt * 16 + (lane >> 2);
                    c0[d0] = o[nt][mt][0] * fac[nt][0];
                    c1[d0] = o[nt][mt][1] * fac[nt][1];
                    c0[d0 + 8] = o[nt][mt][2] * fac[nt][0];
                    c1[d0 + 8] = o[nt][mt][3] * fac[nt][1];
                }
            }
            named_bar_sync(2, kConsumerThreads);
            // this CTA's (m, l) of every head to every CTA of the cluster
            for (uint32_t idx = tid; idx < C * HP; idx += kConsumerThreads) {
                const uint32_t r = idx / HP, g = idx - r * HP;
                float m_all = kNegSentinel;
#pragma unroll
                for (uint32_t w = 0; w < kConsumerWarps; ++w) m_all = fmaxf(m_all, ml_s[(w * HP + g) * 2]);
                float l_all = 0.f;
#pragma unroll
                for (uint32_t w = 0; w < kConsumerWarps; ++w)
                    l_all += ml_s[(w * HP + g) * 2 + 1] * fast_exp2(ml_s[(w * HP + g) * 2] - m_all);
                st_cluster_f2(cluster_map_shared(recv_ml_addr + (crank * HP + g) * 8, r), m_all, l_all);
            }
            // four heads of one dim per thread: one 16-byte store into the owner's shared memory
            for (uint32_t e = tid; e < (HP / 4) * D; e += kConsumerThreads) {
                const uint32_t gq = e / D, d = e - gq * D;
                if (gq * 4 >= G) continue;  // padded heads are never read
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (uint32_t w = 0; w < kConsumerWarps; ++w) {
                    const float *c4 = cf + (w * HP + gq * 4) * kFS + d;
                    acc.x += c4[0];
                    acc.y += c4[kFS];
                    acc.z += c4[2 * kFS];
                    acc.w += c4[3 * kFS];
                }
                const uint32_t owner = d / own_dims, dl = d - owner * own_dims;
                st_cluster_f4(cluster_map_shared(recv_acc_addr + ((crank * own_dims + dl) * HP + gq * 4) * 4, owner), acc);
            }
        }
        // The four warps' accumulators meet in shared memory, one half of the head dimension per
        // pass (the buffer is half-width so that two CTAs fit one SM).
#pragma unroll
        for (int hp = 0; hp < (cl ? 0 : 2); ++hp) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint32_t h0 = nt * 8 + 2 * (lane & 3);
                float *c0 = comb + (warp * HP + h0) * S::kCombStride;
                float *c1 = c0 + S::kCombStride;
#pragma unroll
                for (int mh = 0; mh < D / 32; ++mh) {
                    const int mt = hp * (D / 32) + mh;
                    const uint32_t d0 = mh * 16 + (lane >> 2);
                    c0[d0] = o[nt][mt][0] * fac[nt][0];
                    c1[d0] = o[nt][mt][1] * fac[nt][1];
                    c0[d0 + 8] = o[nt][mt][2] * fac[nt][0];
                    c1[d0 + 8] = o[nt][mt][3] * fac[nt][1];
                }
            }
            named_bar_sync(2, kConsumerThreads);
            for (uint32_t e = tid; e < HP * (D / 2); e += kConsumerThreads) {
                const uint32_t g = e / (D / 2), dd = e - g * (D / 2), d = hp * (D / 2) + dd;
                float m_all = kNegSentinel;
#pragma unroll
                for (uint32_t w = 0; w < kConsumerWarps; ++w) m_all = fmaxf(m_all, ml_s[(w * HP + g) * 2]);
                float l_all = 0.f, acc = 0.f;
#pragma unroll
                for (uint32_t w = 0; w < kConsumerWarps; ++w) {
                    l_all += ml_s[(w * HP + g) * 2 + 1] * fast_exp2(ml_s[(w * HP + g) * 2] - m_all);
                    acc += comb[(w * HP + g) * S::kCombStride + dd];
                }
                const uint32_t h = it.kvh * G + g;
                if (!direct) {
                    p.part_acc[((size_t)it.slot * HP + g) * D + d] = acc;
                    if (d == 0) {
                        p.part_ml[((size_t)it.slot * HP + g) * 2] = m_all * kLn2;
                        p.part_ml[((size_t)it.slot * HP + g) * 2 + 1] = l_all;
                    }
                } else if (g < G) {
                    if (p.push_world) {
                        const size_t rows = (size_t)p.batch * p.n_heads, rowi = (size_t)it.seq * p.n_heads + h;
                        for (uint32_t r = 0; r < p.push_world; ++r) {
                            push_store(p, r, rowi * D + d, acc);
                            if (d == 0) {
                                push_store(p, r, rows * D + rowi, m_all * kLn2);
                                push_store(p, r, rows * D + rows + rowi, l_all);
                            }
                        }
                    } else if (partial_out) {
                        p.out_acc[((size_t)it.seq * p.n_heads + h) * D + d] = acc;
                        if (d == 0) {
                            p.out_m[(size_t)it.seq * p.n_heads + h] = m_all * kLn2;
                            p.out_l[(size_t)it.seq * p.n_heads + h] = l_all;
                        }
                    } else {
                        const bool ok = (fabsf(l_all) <= 3.0e38f) && fabsf(l_all) > 1e-6f;
                        float r = ok ? acc / l_all : acc;
                        if (!(fabsf(r) <= 3.0e38f)) r = 0.f;
                        p.out[(size_t)it.seq * p.out_stride_b + (size_t)h * p.out_stride_h + d] = __float2half_rn(r);
                    }
                }
            }
            if (hp == 0) named_bar_sync(1, kConsumerThreads);  // pass 1 reuses the buffer
        }
        if (cl) {
            // ---- the cluster's CTAs meet: every store above has landed once all of them have arrived ----
            __syncwarp();
            cluster_arrive_release();
            cluster_wait_acquire();
            const float *racc = reinterpret_cast<const float *>(smem + S::kOffRecv);
            const float2 *rml = reinterpret_cast<const float2 *>(smem + S::kOffRecv + S::kRecvAccBytes);
            for (uint32_t col = tid; col < own_dims * HP; col += kConsumerThreads) {  // (dim, head) columns this CTA owns
                const uint32_t g = col % HP, dl = col / HP, d = crank * own_dims + dl;
                if (g >= G) continue;
                float mx = kNegSentinel;
#pragma unroll 4
                for (uint32_t r = 0; r < C; ++r) mx = fmaxf(mx, rml[r * HP + g].x);
                float lt = 0.f, acc = 0.f;
#pragma unroll 4
                for (uint32_t r = 0; r < C; ++r) {
                    const float2 ml = rml[r * HP + g];
                    const float w = fast_exp2(ml.x - mx);
                    lt += ml.y * w;
                    acc += racc[(r * own_dims + dl) * HP + g] * w;
                }
                const uint32_t h = it.kvh * G + g;
                if (!direct) {
                    // the cluster's partial of the unit; the CTA that completes the unit merges (ticket below)
                    p.part_acc[((size_t)it.slot * HP + g) * D + d] = acc;
                    if (d == 0) *reinterpret_cast<float2 *>(p.part_ml + ((size_t)it.slot * HP + g) * 2) = make_float2(mx * kLn2, lt);
                } else if (p.push_world) {
                    const size_t rows = (size_t)p.batch * p.n_heads, rowi = (size_t)it.seq * p.n_heads + h;
                    for (uint32_t r = 0; r < p.push_world; ++r) {
                        push_store(p, r, rowi * D + d, acc);
                        if (d == 0) {
                            push_store(p, r, rows * D + rowi, mx * kLn2);
                            push_store(p, r, rows * D + rows + rowi, lt);
                        }
                    }
                } else if (partial_out) {
                    p.out_acc[((size_t)it.seq * p.n_heads + h) * D + d] = acc;
                    if (d == 0) {
                        p.out_m[(size_t)it.seq * p.n_heads + h] = mx * kLn2;
                        p.out_l[(size_t)it.seq * p.n_heads + h] = lt;
                    }
                } else {
                    const bool ok = (fabsf(lt) <= 3.0e38f) && fabsf(lt) > 1e-6f;
                    float r1 = ok ? acc / lt : acc;  // decode rule: the sum itself when l is tiny
                    if (!(fabsf(r1) <= 3.0e38f)) r1 = 0.f;
                    p.out[(size_t)it.seq * p.out_stride_b + (size_t)h * p.out_stride_h + d] = __float2half_rn(r1);
                }
            }
            if (direct) {
                if (!p.push_world) continue;  // nobody reads another CTA's shared memory after the barrier: done
                // Every CTA's share of the unit must be in the peers' receive blocks before the first CTA announces
                // it.  The owners' stores happen before this barrier, the barrier before the system-scope fence that
                // the announcing CTA executes in front of its counter updates (push_signal_and_merge): fences are
                // cumulative, so one fence orders all sixteen CTAs' stores - and a system-scope fence costs about
                // 5 us here whatever is outstanding, which is why the owners do not each execute one of their own.
                // (Tagged words need neither: the merging CTA reads until every word of every block, this cluster's
                // own included, carries the step's tag.)
                if (!p.push_tagged) {
                    __syncwarp();
                    cluster_arrive_release();
                    cluster_wait_acquire();
                }
                if (crank == 0) push_signal_and_merge<D>(p, it, tid, flags);
                continue;
            }
            // not direct: every CTA of every cluster of the unit takes a ticket below; the last one merges
        } else if (direct) {
            if (p.push_world) push_signal_and_merge<D>(p, it, tid, flags);
            continue;
        }

        // ---- ticket: the CTA that completes the unit merges its partials ---------------
        __threadfence();
        named_bar_sync(1, kConsumerThreads);
        if (tid == 0) {
            const uint32_t old = atomicAdd(p.counters + it.unit, 1u);
            // cluster form: every CTA of the unit's clusters arrives with its own share of a partial
            const uint32_t last = (old + 1 == it.n_parts * C) ? 1u : 0u;
            if (last) p.counters[it.unit] = 0;  // ready for the next launch
            flags[1] = last;
        }
        named_bar_sync(2, kConsumerThreads);
        if (!flags[1]) continue;
        __threadfence();
        // Merge (flash_prefill.metal:843-888), arranged so that the loads of one round trip are all
        // in flight together: this runs at the end of a CTA's work, where latency is not hidden.
        constexpr uint32_t kMergeCap = 64;                       // parts whose m is cached in smem
        constexpr uint32_t kPerHead = kConsumerThreads / HP;     // threads per head in pass 1
        float *msv = comb;                                       // [kMergeCap][HP]
        float *red = comb + kMergeCap * HP;                      // [threads][2]
        {
            const uint32_t g1 = tid % HP;
            float m_loc = kNegSentinel, l_loc = 0.f;
            for (uint32_t sp = tid / HP; sp < it.n_parts; sp += kPerHead) {
                const float2 ml = __ldcg(reinterpret_cast<const float2 *>(p.part_ml) + (size_t)(it.first_slot + sp) * HP + g1);
                if (sp < kMergeCap) msv[sp * HP + g1] = ml.x;
                const float mn = fmaxf(m_loc, ml.x);
                l_loc = l_loc * __expf(m_loc - mn) + (ml.y > 0.f ? ml.y * __expf(ml.x - mn) : 0.f);
                m_loc = mn;
            }
            red[tid * 2] = m_loc;
            red[tid * 2 + 1] = l_loc;
        }
        named_bar_sync(1, kConsumerThreads);
        // Pass 2: one float4 column of one real head per thread and round, kMergeFlight parts in flight.
        const uint32_t cols4 = G * (D / 4);
        for (uint32_t c4 = tid; c4 < cols4; c4 += kConsumerThreads) {
            const uint32_t g2 = c4 / (D / 4), d0 = (c4 % (D / 4)) * 4;
            float mx = kNegSentinel, lt = 0.f;
#pragma unroll
            for (uint32_t j = 0; j < kPerHead; ++j) mx = fmaxf(mx, red[(j * HP + g2) * 2]);
#pragma unroll
            for (uint32_t j = 0; j < kPerHead; ++j) lt += red[(j * HP + g2) * 2 + 1] * __expf(red[(j * HP + g2) * 2] - mx);
            // Rounds of F loads in flight; parts are added in order, so F does not change the bits.  Units
            // cut in a few parts (the batched step) take the narrow form: a round costs F slots whether
            // they are used or not.
            auto accumulate = [&](auto flight) {
                constexpr uint32_t F = decltype(flight)::value;
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
                for (uint32_t s0 = 0; s0 < it.n_parts; s0 += F) {
                    float4 v[F];
                    float w[F];
#pragma unroll
                    for (uint32_t j = 0; j < F; ++j) {
                        const uint32_t sp = s0 + j;
                        if (sp < it.n_parts) {
                            const size_t sl = it.first_slot + sp;
                            v[j] = __ldcg(reinterpret_cast<const float4 *>(p.part_acc + (sl * HP + g2) * D + d0));
                            const float ms = sp < kMergeCap ? msv[sp * HP + g2] : __ldcg(p.part_ml + (sl * HP + g2) * 2);
                            w[j] = __expf(ms - mx);
                        } else {
                            v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                            w[j] = 0.f;
                        }
                    }
#pragma unroll
                    for (uint32_t j = 0; j < F; ++j) {
                        a.x += v[j].x * w[j];
                        a.y += v[j].y * w[j];
                        a.z += v[j].z * w[j];
                        a.w += v[j].w * w[j];
                    }
                }
                return a;
            };
            const float4 acc = it.n_parts <= kMergeFlightFew ? accumulate(std::integral_constant<uint32_t, kMergeFlightFew>{})
                                                             : accumulate(std::integral_constant<uint32_t, kMergeFlight>{});
            const uint32_t h = it.kvh * G + g2;
            if (p.push_world) {
                const size_t rows = (size_t)p.batch * p.n_heads, rowi = (size_t)it.seq * p.n_heads + h;
                for (uint32_t r = 0; r < p.push_world; ++r) {
                    if (p.push_tagged) {
                        push_store(p, r, rowi * D + d0, acc.x);
                        push_store(p, r, rowi * D + d0 + 1, acc.y);
                        push_store(p, r, rowi * D + d0 + 2, acc.z);
                        push_store(p, r, rowi * D + d0 + 3, acc.w);
                    } else {
                        *reinterpret_cast<float4 *>(p.push_dst[r] + rowi * D + d0) = acc;
                    }
                    if (d0 == 0) {
                        push_store(p, r, rows * D + rowi, mx);
                        push_store(p, r, rows * D + rows + rowi, lt);
                    }
                }
            } else if (partial_out) {
                *reinterpret_cast<float4 *>(p.out_acc + ((size_t)it.seq * p.n_heads + h) * D + d0) = acc;
                if (d0 == 0) {
                    p.out_m[(size_t)it.seq * p.n_heads + h] = mx;
                    p.out_l[(size_t)it.seq * p.n_heads + h] = lt;
                }
            } else {
                const bool ok = (fabsf(lt) <= 3.0e38f) && fabsf(lt) > 1e-6f;
                const float inv = ok ? 1.0f / lt : 0.f;  // merge rule: flash_prefill.metal:861
                float r[4] = {acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv};
                __half *dst = p.out + (size_t)it.seq * p.out_stride_b + (size_t)h * p.out_stride_h + d0;
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) {
                    if (!(fabsf(r[i]) <= 3.0e38f)) r[i] = 0.f;
                    dst[i] = __float2half_rn(r[i]);
                }
            }
        }
        if (p.push_world) push_signal_and_merge<D>(p, it, tid, flags);
    }
}

// Per device and instantiation, once: the dynamic shared memory limit, and the largest cluster the kernel can
// be launched with (16 needs the non-portable opt-in; 8 is portable; 0 if not even that is schedulable).
template <int D, int NT, int STAGES, int MINB>
mf_status configure_one(MfContext *ctx, uint32_t *max_cluster_out)
{
    using S = Smem<D, NT, STAGES, false>;
    using SC = Smem<D, NT, STAGES, true>;
    static_assert(MINB * (SC::kDynamic + 1024) <= 228 * 1024, "CTAs per SM do not fit shared memory");
    static bool configured[64] = {};
    static uint32_t max_cluster[64] = {};
    auto kern = decode_kernel<D, NT, STAGES, MINB, false>;
    auto kern_cl = decode_kernel<D, NT, STAGES, MINB, true>;
    const int dev = ctx->device;
    if (dev < 0 || dev >= 64) return fail(ctx, MF_ERR_INVALID_OPERATION, "device index %d", dev);
    if (!configured[dev]) {
        mf_status st = check_cuda(
            ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kDynamic),
            "cudaFuncSetAttribute(decode)");
        if (st != MF_OK) return st;
        st = check_cuda(ctx, cudaFuncSetAttribute(kern_cl, cudaFuncAttributeMaxDynamicSharedMemorySize, SC::kDynamic),
                        "cudaFuncSetAttribute(decode, cluster form)");
        if (st != MF_OK) return st;
        int resident = 0, resident_cl = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kern, (int)kThreads, S::kDynamic) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident_cl, kern_cl, (int)kThreads, SC::kDynamic) != cudaSuccess ||
            resident < MINB || resident_cl < MINB)
            return fail(ctx, MF_ERR_CUDA, "decode kernel: %d / %d CTAs per SM fit, the variant is built for %d", resident,
                        resident_cl, MINB);
        // The largest cluster size the device takes, and how many clusters of 16 and of 8 CTAs it holds at once
        // (packed into the value: bits 0-7 the size, 8-15 the count for 16, 16-23 the count for 8): a launch whose
        // clusters are not all resident runs them in waves.
        uint32_t best = 0, fit16 = 0, fit8 = 0;
        const bool wide = cudaFuncSetAttribute(kern_cl, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
        for (uint32_t c : {16u, 8u}) {
            if (c == 16 && !wide) continue;
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3(c);
            cfg.blockDim = dim3(kThreads);
            cfg.dynamicSmemBytes = SC::kDynamic;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = c;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, kern_cl, &cfg) == cudaSuccess && n >= 1) {
                if (!best) best = c;
                (c == 16 ? fit16 : fit8) = (uint32_t)std::min(n, 255);
            }
        }
        (void)cudaGetLastError();  // a refused query is an answer, not an error of this call
        max_cluster[dev] = best | (fit16 << 8) | (fit8 << 16);
        configured[dev] = true;
    }
    if (max_cluster_out) *max_cluster_out = max_cluster[dev];
    return MF_OK;
}

template <int D, int NT, int STAGES, int MINB>
mf_status launch_one(MfContext *ctx, const CUtensorMap &tm_k, const CUtensorMap &tm_v,
                     DecodeParams &p, uint32_t n_ctas, const void *writes_k, const void *writes_v)
{
    const bool clustered = p.cluster_size > 1;
    auto kern = clustered ? decode_kernel<D, NT, STAGES, MINB, true> : decode_kernel<D, NT, STAGES, MINB, false>;
    const uint32_t smem_bytes = clustered ? Smem<D, NT, STAGES, true>::kDynamic : Smem<D, NT, STAGES, false>::kDynamic;
    mf_status st = configure_one<D, NT, STAGES, MINB>(ctx, nullptr);
    if (st != MF_OK) return st;
    if (p.cluster_size > 1 && n_ctas % p.cluster_size != 0)
        return fail(ctx, MF_ERR_INVALID_OPERATION, "decode: %u CTAs in clusters of %u", n_ctas, p.cluster_size);
    if (ctx->overlap_launches || p.cluster_size > 1) {
        const bool programmatic = ctx->overlap_launches != 0;
        p.strict_release = (programmatic && ctx->next_launch_strict()) ? 1u : 0u;
        p.release_late = (clustered && !p.strict_release) ? 1u : 0u;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(n_ctas);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = smem_bytes;
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[2];
        unsigned n_attr = 0;
        if (programmatic) {
            attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
            ++n_attr;
        }
        if (p.cluster_size > 1) {
            attr[n_attr].id = cudaLaunchAttributeClusterDimension;
            attr[n_attr].val.clusterDim.x = p.cluster_size;
            attr[n_attr].val.clusterDim.y = 1;
            attr[n_attr].val.clusterDim.z = 1;
            ++n_attr;
        }
        cfg.attrs = attr;
        cfg.numAttrs = n_attr;
        cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tm_k, tm_v, p);
        if (e != cudaSuccess) return fail(ctx, MF_ERR_CUDA, "launch decode_kernel: %s", cudaGetErrorString(e));
        ++ctx->launches;
        if (programmatic) ctx->note_programmatic_launch(p.strict_release != 0, writes_k, writes_v);
        return MF_OK;
    }
    kern<<<n_ctas, kThreads, smem_bytes, ctx->stream>>>(tm_k, tm_v, p);
    return check_launch(ctx, "decode_kernel");
}

}  // namespace


uint32_t decode_ctas_per_sm(const MfContext *ctx, uint32_t head_dim, uint32_t group)
{
    if (group > 8) return 1;
    if (head_dim == 128 && ctx && ctx->decode_stages == 6) return 1;
    return 2;
}

// Number of CTAs for `total` tiles: as many as are resident, but a span shorter than eight
// tiles mostly pays for its own boundary (q load, combine, partial write, a longer merge), so
// small problems get one CTA per SM.
// A CTA that straddles two units pays the per-item work twice (q staging, combine, partial write,
// ticket: about 3 us), and the launch ends with the slowest CTA.  When the launch is short - few tiles
// per CTA - and there are several CTAs per unit anyway, cutting every unit on its own is cheaper than
// perfectly equal spans.
constexpr uint32_t kAlignMaxSpan = 32;   // tiles per CTA up to which units are cut separately
constexpr uint32_t kAlignMinParts = 4;   // ... given at least this many CTAs per unit

uint32_t decode_max_cluster(MfContext *ctx, uint32_t head_dim, uint32_t group)
{
    if (!ctx || ctx->decode_clusters == 1) return 0;
    const uint32_t nt = (group + 7) / 8;
    uint32_t c = 0;
    mf_status st = MF_ERR_OPERATION_NOT_SUPPORTED;
    if (head_dim == 128 && nt == 1 && ctx->decode_stages == 6) st = configure_one<128, 1, 6, 1>(ctx, &c);
    else if (head_dim == 128 && nt == 1) st = configure_one<128, 1, 3, 2>(ctx, &c);
    else if (head_dim == 128 && nt == 2) st = configure_one<128, 2, 5, 1>(ctx, &c);
    else if (head_dim == 64 && nt == 1) st = configure_one<64, 1, 6, 2>(ctx, &c);
    else if (head_dim == 64 && nt == 2) st = configure_one<64, 2, 8, 1>(ctx, &c);
    return st == MF_OK ? c : 0;
}

// Cluster form of a short launch: the `per_unit` CTAs a unit can have are arranged as k clusters of c CTAs, c a
// power of two up to max_cluster.  A large c leaves few partials to merge through memory (none when k == 1);
// a small c wastes fewer CTAs when per_unit is not a multiple.  The largest c that keeps at least 85 % of the
// CTAs the best choice would use is taken.
void cluster_shape(uint32_t per_unit, uint32_t tiles_per_unit, uint32_t units, uint32_t max_cluster_packed, uint32_t *c_out,
                   uint32_t *k_out)
{
    *c_out = *k_out = 0;
    const uint32_t max_cluster = max_cluster_packed & 0xFFu, fit16 = (max_cluster_packed >> 8) & 0xFFu,
                   fit8 = (max_cluster_packed >> 16) & 0xFFu;
    // all clusters of the launch resident at once (sizes below 8 always are, for the launches this form is used for)
    auto resident = [&](uint32_t c, uint32_t k) {
        const uint32_t fit = c == 16 ? fit16 : (c == 8 ? fit8 : 0xFFFFu);
        return fit == 0 || (uint64_t)k * units <= fit;
    };
    uint32_t best = 0;
    for (uint32_t c = 2; c <= max_cluster; c *= 2) {
        const uint32_t k = std::min(per_unit / c, tiles_per_unit / c);
        if (resident(c, k)) best = std::max(best, k * c);
    }
    if (!best) return;
    for (uint32_t c = max_cluster; c >= 2; c /= 2) {
        const uint32_t k = std::min(per_unit / c, tiles_per_unit / c);
        if (k && resident(c, k) && k * c * 100 >= best * 85) {
            *c_out = c;
            *k_out = k;
            return;
        }
    }
}

UniformSplit uniform_split(uint32_t units, uint32_t tiles_per_unit, uint32_t n_splits, uint32_t want_ctas,
                           uint32_t max_cluster)
{
    UniformSplit r{};
    const uint32_t T = tiles_per_unit;
    const uint64_t total = (uint64_t)units * T;
    if (n_splits > 0) {
        r.span = std::max(1u, (T + n_splits - 1) / n_splits);
        r.parts = (T + r.span - 1) / r.span;
        r.n_ctas = units * r.parts;
        return r;
    }
    const uint32_t flat_span = std::max<uint32_t>(1, (uint32_t)((total + want_ctas - 1) / want_ctas));
    if (max_cluster >= 2 && want_ctas >= kAlignMinParts * units && flat_span <= kAlignMaxSpan) {
        uint32_t c = 0, k = 0;
        cluster_shape(want_ctas / units, T, units, max_cluster, &c, &k);
        if (c) {
            r.cluster = c;
            r.span = (T + k - 1) / k;
            r.parts = (T + r.span - 1) / r.span;  // ranges (clusters) per unit
            r.n_ctas = units * r.parts * c;
            return r;
        }
    }
    if (want_ctas >= kAlignMinParts * units && flat_span <= kAlignMaxSpan) {
        const uint32_t parts = std::min(want_ctas / units, T);
        r.span = (T + parts - 1) / parts;
        r.parts = (T + r.span - 1) / r.span;
        r.n_ctas = units * r.parts;
        return r;
    }
    r.span = flat_span;
    r.parts = 0;
    r.n_ctas = (uint32_t)((total + flat_span - 1) / flat_span);
    return r;
}

uint32_t decode_cta_target(uint32_t sm_count, uint32_t ctas_per_sm, uint64_t total)
{
    const uint64_t resident = (uint64_t)sm_count * ctas_per_sm;
    uint64_t want = resident;
    if (ctas_per_sm > 1 && total < resident * 8) want = sm_count;
    if (want > total) want = total;
    return (uint32_t)(want ? want : 1);
}

mf_status launch_decode(MfContext *ctx, const CUtensorMap &tm_k, const CUtensorMap &tm_v,
                        DecodeParams &p, uint32_t head_dim, uint32_t n_ctas, const void *writes_k,
                        const void *writes_v)
{
    const uint32_t nt = (p.group + 7) / 8;
    if (nt > 2) return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "decode: group size %u > 16", p.group);
    // Groups of up to 8 query heads: two CTAs per SM, each with a short ring, so that one CTA's
    // span boundary (combine, partial write, merge, q load) overlaps the other's tile stream.
    if (head_dim == 128) {
        if (nt == 1 && ctx->decode_stages == 6) return launch_one<128, 1, 6, 1>(ctx, tm_k, tm_v, p, n_ctas, writes_k, writes_v);
        return nt == 1 ? launch_one<128, 1, 3, 2>(ctx, tm_k, tm_v, p, n_ctas, writes_k, writes_v)
                       : launch_one<128, 2, 5, 1>(ctx, tm_k, tm_v, p, n_ctas, writes_k, writes_v);
    }
    if (head_dim == 64) {
        return nt == 1 ? launch_one<64, 1, 6, 2>(ctx, tm_k, tm_v, p, n_ctas, writes_k, writes_v)
                       : launch_one<64, 2, 8, 1>(ctx, tm_k, tm_v, p, n_ctas, writes_k, writes_v);
    }
    return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "Flash Decode only supports head_dim=64 or 128, got %u",
                head_dim);
}

void build_decode_plan(const uint32_t *kv_lens, uint32_t batch, uint32_t n_kv_heads,
                       uint32_t max_ctas, std::vector<WorkItem> &items,
                       std::vector<uint32_t> &cta_begin, uint32_t *n_units, uint64_t *total_tiles,
                       uint32_t *cluster_out, uint32_t item_cost)
{
    const uint32_t max_cluster = cluster_out ? *cluster_out : 0;
    if (cluster_out) *cluster_out = 0;
    items.clear();
    cta_begin.clear();
    uint64_t total = 0;
    for (uint32_t b = 0; b < batch; ++b) total += (uint64_t)((kv_lens[b] + kTileKeys - 1) / kTileKeys) * n_kv_heads;
    *total_tiles = total;
    *n_units = batch * n_kv_heads;
    if (total == 0) {
        cta_begin.push_back(0);
        return;
    }
    const uint32_t n_ctas = (uint32_t)(total < max_ctas ? total : max_ctas);
    // Short launch with several CTAs per unit: cut every unit on its own (see uniform_split).
    uint32_t live_units = 0;
    for (uint32_t b = 0; b < batch; ++b) live_units += kv_lens[b] ? n_kv_heads : 0;
    if (n_ctas >= kAlignMinParts * live_units && (total + n_ctas - 1) / n_ctas <= kAlignMaxSpan) {
        // Cluster form, when every live sequence has the same number of tiles (one sequence, or equal lengths):
        // each unit is cut into k ranges, one item and one cluster of c CTAs per range.
        uint32_t same_tiles = 0;
        bool same = max_cluster >= 2;
        for (uint32_t b = 0; b < batch && same; ++b) {
            const uint32_t tiles = (kv_lens[b] + kTileKeys - 1) / kTileKeys;
            if (!tiles) continue;
            if (same_tiles && tiles != same_tiles) same = false;
            same_tiles = tiles;
        }
        uint32_t c = 0, k = 0;
        if (same && same_tiles) cluster_shape(n_ctas / live_units, same_tiles, live_units, max_cluster, &c, &k);
        if (c) {
            const uint32_t span = (same_tiles + k - 1) / k, ranges = (same_tiles + span - 1) / span;
            uint32_t slot = 0;
            for (uint32_t b = 0; b < batch; ++b) {
                if (!kv_lens[b]) continue;
                for (uint32_t kh = 0; kh < n_kv_heads; ++kh) {
                    const uint32_t first_slot = slot;
                    for (uint32_t ri = 0; ri < ranges; ++ri) {
                        WorkItem it{};
                        it.seq = b;
                        it.kvh = kh;
                        it.tile_begin = ri * span;
                        it.tile_end = std::min(same_tiles, it.tile_begin + span);
                        it.slot = slot++;
                        it.unit = b * n_kv_heads + kh;
                        it.first_slot = first_slot;
                        it.n_parts = ranges;
                        cta_begin.push_back((uint32_t)items.size());
                        items.push_back(it);
                    }
                }
            }
            cta_begin.push_back((uint32_t)items.size());
            *cluster_out = c;
            return;
        }
        // Cluster form for sequences of different lengths: clusters of ONE size c, every unit cut into ranges of about
        // equal length with one cluster per range, so that a unit's CTAs combine through distributed shared memory
        // and only the ranges of a long unit (a few) meet through partials and a ticket.  Every unit needs at least c
        // tiles.  Measured on batches of 2, 4 and 8 sequences of 512 to 16384 tokens: what a launch costs is less the
        // longest share of a CTA than the tickets of the units cut into several ranges (every CTA of every such
        // cluster takes one), so the largest c whose longest share stays within 1.6x of the best c's is taken, and
        // clusters of 16 only when no unit needs a second range.
        if (max_cluster >= 2) {
            const uint32_t c_max = max_cluster & 0xFFu, fit16 = (max_cluster >> 8) & 0xFFu, fit8 = (max_cluster >> 16) & 0xFFu;
            auto ranges_for = [&](uint32_t cc, std::vector<uint32_t> &r) -> uint32_t {  // returns tiles per CTA, 0: not possible
                uint32_t n_cl = n_ctas / cc;
                const uint32_t fit = cc == 16 ? fit16 : (cc == 8 ? fit8 : 0u);
                if (fit) n_cl = std::min(n_cl, fit);
                if (n_cl < live_units) return 0;
                r.assign(batch, 0);
                uint64_t used = 0;
                for (uint32_t b = 0; b < batch; ++b) {
                    const uint32_t tiles = (kv_lens[b] + kTileKeys - 1) / kTileKeys;
                    if (!tiles) continue;
                    if (tiles < cc) return 0;
                    const uint64_t want = (uint64_t)tiles * n_cl / total;
                    r[b] = (uint32_t)std::min<uint64_t>(std::max<uint64_t>(want, 1), tiles / cc);
                    used += (uint64_t)r[b] * n_kv_heads;
                }
                if (used > n_cl) return 0;
                for (;;) {  // clusters left over go to the sequences whose ranges are longest
                    uint32_t pick = batch;
                    double longest = 0.0;
                    for (uint32_t b = 0; b < batch; ++b) {
                        const uint32_t tiles = (kv_lens[b] + kTileKeys - 1) / kTileKeys;
                        if (!tiles || r[b] >= tiles / cc) continue;
                        const double len = (double)tiles / r[b];
                        if (len > longest) {
                            longest = len;
                            pick = b;
                        }
                    }
                    if (pick == batch || used + n_kv_heads > n_cl) break;
                    ++r[pick];
                    used += n_kv_heads;
                }
                uint32_t worst = 0;
                for (uint32_t b = 0; b < batch; ++b) {
                    const uint32_t tiles = (kv_lens[b] + kTileKeys - 1) / kTileKeys;
                    if (!tiles) continue;
                    const uint32_t span = (tiles + r[b] - 1) / r[b];
                    worst = std::max(worst, (span + cc - 1) / cc);
                }
                return worst;
            };
            std::vector<uint32_t> r, r_best;
            uint32_t best_share = 0, c_best = 0;
            for (uint32_t cc = 2; cc <= c_max; cc *= 2) {
                const uint32_t share = ranges_for(cc, r);
                if (share && (!best_share || share < best_share)) best_share = share;
            }
            for (uint32_t cc = c_max; cc >= 2 && best_share; cc /= 2) {
                const uint32_t share = ranges_for(cc, r);
                if (cc > 8 && share && *std::max_element(r.begin(), r.end()) > 1) continue;
                if (share && share * 100 <= best_share * 160) {
                    c_best = cc;
                    r_best = r;
                    break;
                }
            }
            if (c_best) {
                uint32_t slot = 0;
                for (uint32_t b = 0; b < batch; ++b) {
                    const uint32_t tiles = (kv_lens[b] + kTileKeys - 1) / kTileKeys;
                    if (!tiles) continue;
                    // ranges of equal length (the first `rem_t` one tile longer): none shorter than c tiles
                    const uint32_t ranges = r_best[b], base_t = tiles / ranges, rem_t = tiles % ranges;
                    for (uint32_t kh = 0; kh < n_kv_heads; ++kh) {
                        const uint32_t first_slot = slot;
                        uint32_t t = 0;
                        for (uint32_t ri = 0; ri < ranges; ++ri) {
                            WorkItem it{};
                            it.seq = b;
                            it.kvh = kh;
                            it.tile_begin = t;
                            it.tile_end = t + base_t + (ri < rem_t ? 1u : 0u);
                            t = it.tile_end;
                            it.slot = slot++;
                            it.unit = b * n_kv_heads + kh;
                            it.first_slot = first_slot;
                            it.n_parts = ranges;
                            cta_begin.push_back((uint32_t)items.size());
                            items.push_back(it);
                        }
                    }
                }
                cta_begin.push_back((uint32_t)items.size());
                *cluster_out = c_best;
                return;
            }
        }
        // CTAs per unit in proportion to its tiles, at least one, never more than its tiles
        std::vector<uint32_t> parts(batch, 0);  // per sequence: the same for each of its kv heads
        uint64_t used = 0;
        for (uint32_t b = 0; b < batch; ++b) {
            const uint32_t tiles = (kv_lens[b] + kTileKeys - 1) / kTileKeys;
            if (!tiles) continue;
            uint64_t want = (uint64_t)tiles * n_ctas / total;
            parts[b] = (uint32_t)std::min<uint64_t>(std::max<uint64_t>(want, 1), tiles);
            used += (uint64_t)parts[b] * n_kv_heads;
        }
        // hand the CTAs left over to the sequences whose ranges are longest
        for (;;) {
            uint32_t best = batch;
            double best_len = 0.0;
            for (uint32_t b = 0; b < batch; ++b) {
                const uint32_t tiles = (kv_lens[b] + kTileKeys - 1) / kTileKeys;
                if (!tiles || parts[b] >= tiles) continue;
                const double len = (double)tiles / parts[b];
                if (len > best_len) {
                    best_len = len;
                    best = b;
                }
            }
            if (best == batch || used + n_kv_heads > n_ctas) break;
            ++parts[best];
            used += n_kv_heads;
        }
        uint32_t slot = 0;
        for (uint32_t b = 0; b < batch; ++b) {
            const uint32_t tiles = (kv_lens[b] + kTileKeys - 1) / kTileKeys;
            if (!tiles) continue;
            const uint32_t np = parts[b], base_t = tiles / np, rem_t = tiles % np;
            for (uint32_t kh = 0; kh < n_kv_heads; ++kh) {
                const uint32_t first_slot = slot;
                uint32_t t = 0;
                for (uint32_t pi = 0; pi < np; ++pi) {
                    const uint32_t take = base_t + (pi < rem_t ? 1 : 0);
                    WorkItem it{};
                    it.seq = b;
                    it.kvh = kh;
                    it.tile_begin = t;
                    it.tile_end = t + take;
                    it.slot = slot++;
                    it.unit = b * n_kv_heads + kh;
                    it.first_slot = first_slot;
                    it.n_parts = np;
                    cta_begin.push_back((uint32_t)items.size());
                    items.push_back(it);
                    t += take;
                }
            }
        }
        cta_begin.push_back((uint32_t)items.size());
        return;
    }
    // Long launch: CTAs take consecutive tiles across unit boundaries.  What is equal from CTA to CTA is not the
    // number of tiles but tiles + item_cost * items: every piece of a unit costs a CTA the staging of q, the combine
    // of its warps, a partial and a ticket, for one piece of a unit its merge (5-10 us, the time of `item_cost` tiles), and the launch behind this one
    // cannot start its arithmetic before the slowest CTA has ended.  With equal tile counts the few CTAs that cover
    // three or four short sequences ended 15-20 us after the median one (batch 64, lengths 512-16384).
    const uint64_t c = item_cost;
    auto pieces_fit = [&](uint64_t budget, bool emit) -> uint64_t {
        uint64_t ctas = 0, room = 0;
        uint32_t slot = 0;
        for (uint32_t b = 0; b < batch; ++b) {
            const uint32_t tiles = (kv_lens[b] + kTileKeys - 1) / kTileKeys;
            if (tiles == 0) continue;
            for (uint32_t kh = 0; kh < n_kv_heads; ++kh) {
                const uint32_t first_slot = slot;
                const size_t first_item = items.size();
                uint32_t t = 0;
                while (t < tiles) {
                    // a piece shorter than a few tiles is not worth its fixed cost: rather leave the room unused
                    const uint64_t least = std::min<uint64_t>(kMinPieceTiles, tiles - t);
                    if (room < c + least) {
                        ++ctas;
                        room = budget;
                        if (emit) cta_begin.push_back((uint32_t)items.size());
                    }
                    const uint32_t take = (uint32_t)std::min<uint64_t>(tiles - t, room - c);
                    if (emit) {
                        WorkItem it{};
                        it.seq = b;
                        it.kvh = kh;
                        it.tile_begin = t;
                        it.tile_end = t + take;
                        it.slot = slot;
                        it.unit = b * n_kv_heads + kh;
                        it.first_slot = first_slot;
                        items.push_back(it);
                    }
                    ++slot;
                    t += take;
                    room -= take + c;
                }
                if (emit) {
                    const uint32_t parts = (uint32_t)(items.size() - first_item);
                    for (size_t i = first_item; i < items.size(); ++i) items[i].n_parts = parts;
                }
            }
        }
        return ctas;
    };
    // smallest budget with which the pieces fit into n_ctas CTAs
    uint64_t lo = c + 1, hi = total + c * (uint64_t)(*n_units) + c + kMinPieceTiles;
    while (lo < hi) {
        const uint64_t mid = (lo + hi) / 2;
        if (pieces_fit(mid, false) <= n_ctas) hi = mid;
        else lo = mid + 1;
    }
    while (pieces_fit(lo, false) > n_ctas) ++lo;  // (the count is not strictly monotonic in the budget)
    (void)pieces_fit(lo, true);
    while (cta_begin.size() < (size_t)n_ctas + 1) cta_begin.push_back((uint32_t)items.size());
}

}  // namespace mf

// ---------------------------------------------------------------------------------------
// Decode without any allocation: mf_flash_decode_static_scratch.
//
// Some hosts of this library may not allocate device memory at all: an inference server
// that has handed the whole GPU to its own pooling allocator and forbids plug-ins to call
// cudaMalloc, a latency-critical decode loop that cannot afford the device-wide
// synchronisation cudaMalloc / cudaFree imply, or a sandbox that simply denies the call.
// For them the split-KV partials and unit tickets of the decode kernel live in the
// file-scope device array below instead of a cudaMalloc'ed arena.  The array has a fixed,
// modest size; a request that does not fit is refused, never grown.
//
// The array is per device and shared by every call in the process.  It keeps whatever the
// previous call left, so each call clears the words that must start at zero (status and
// tickets) on the caller's stream before its kernel.  Two calls that overlap on the same
// GPU (different streams, or different host threads) race on it: serialise them.
namespace mf {
namespace {

constexpr uint32_t kStaticScratchBytes = 4u << 20;   // whole array, per GPU
constexpr uint32_t kStaticStatusBytes = 256;         // word 0: timeout status of the last call
constexpr uint32_t kStaticTicketBytes = 16u << 10;   // up to 4096 (batch x kv head) units
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

typedef CUresult (*StaticEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct StaticDeviceState {
    bool ready = false;
    unsigned char *scratch = nullptr;  // device address of g_static_scratch on this device
    int sm_count = 0;
    StaticEncodeFn encode = nullptr;
};
StaticDeviceState g_static_state[64];

mf_status static_fail(char *buf, uint32_t len, mf_status code, const char *fmt, unsigned long long a = 0,
                      unsigned long long b = 0)
{
    if (buf && len) snprintf(buf, len, fmt, a, b);
    return code;
}

template <int D, int NT, int STAGES, int MINB>
cudaError_t static_prepare_kernel()
{
    return cudaFuncSetAttribute(decode_kernel<D, NT, STAGES, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                Smem<D, NT, STAGES>::kDynamic);
}

template <int D, int NT, int STAGES, int MINB>
cudaError_t static_launch(const CUtensorMap &tm_k, const CUtensorMap &tm_v, const DecodeParams &p, uint32_t n_ctas,
                          cudaStream_t stream)
{
    decode_kernel<D, NT, STAGES, MINB><<<n_ctas, kThreads, Smem<D, NT, STAGES>::kDynamic, stream>>>(tm_k, tm_v, p);
    return cudaGetLastError();
}

// Once per device, with that device current.  In host code `g_static_scratch` is only a
// stand-in for the symbol: the address a kernel can use comes from cudaGetSymbolAddress.
mf_status static_setup(int device, char *err, uint32_t err_len)
{
    StaticDeviceState &st = g_static_state[device];
    void *ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || !ptr)
        return static_fail(err, err_len, MF_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed (%llu)", (unsigned long long)e);
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess || major != 10)
        return static_fail(err, err_len, MF_ERR_OPERATION_NOT_SUPPORTED, "device is not sm_100 (major %llu)", (unsigned long long)major);
    if (cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || st.sm_count <= 0)
        return static_fail(err, err_len, MF_ERR_CUDA, "cannot read the SM count");
    cudaDriverEntryPointQueryResult q;
    void *fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess || !fn)
        return static_fail(err, err_len, MF_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    st.encode = reinterpret_cast<StaticEncodeFn>(fn);
    if (static_prepare_kernel<128, 1, 3, 2>() != cudaSuccess || static_prepare_kernel<128, 2, 5, 1>() != cudaSuccess ||
        static_prepare_kernel<64, 1, 6, 2>() != cudaSuccess || static_prepare_kernel<64, 2, 8, 1>() != cudaSuccess)
        return static_fail(err, err_len, MF_ERR_CUDA, "cudaFuncSetAttribute(decode) failed");
    st.scratch = static_cast<unsigned char *>(ptr);
    st.ready = true;
    return MF_OK;
}

bool static_encode(const StaticDeviceState &st, const void *base, uint64_t rows, uint32_t cols, CUtensorMap *out)
{
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstride[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64, kTileKeys};
    cuuint32_t estr[2] = {1, 1};
    return st.encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), gdim, gstride, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace
}  // namespace mf

extern "C" mf_status mf_flash_decode_static_scratch(void *cuda_stream, const void *q, const void *k, const void *v,
                                                    void *output, const MfFlashDecodeStrides *s, const SdpaParams *sp,
                                                    uint32_t n_heads, uint32_t batch, char *err, uint32_t err_len)
{
    using namespace mf;
    if (err && err_len) err[0] = 0;
    if (!q || !k || !v || !output || !s || !sp)
        return static_fail(err, err_len, MF_ERR_INPUT_NOT_FOUND, "null tensor or parameter block");
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64)
        return static_fail(err, err_len, MF_ERR_CUDA, "no current CUDA device");
    if (!g_static_state[device].ready) {
        mf_status st = static_setup(device, err, err_len);
        if (st != MF_OK) return st;
    }
    const StaticDeviceState &dst = g_static_state[device];
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);

    // Same contract checks as mf_flash_decode.
    const uint32_t D = sp->head_dim;
    if (D != 64 && D != 128)
        return static_fail(err, err_len, MF_ERR_OPERATION_NOT_SUPPORTED, "Flash Decode only supports head_dim=64 or 128, got %llu", D);
    if (sp->stride_k_s != D || sp->stride_v_s != D)
        return static_fail(err, err_len, MF_ERR_OPERATION_NOT_SUPPORTED, "K/V row stride must equal head_dim");
    if (sp->kv_len == 0 || batch == 0 || n_heads == 0) return MF_OK;
    if (s->q_stride_h == 0 || s->k_stride_h == 0 || s->v_stride_h == 0)
        return static_fail(err, err_len, MF_ERR_INVALID_SHAPE, "zero head stride");
    const uint32_t q_heads = s->q_stride_b / s->q_stride_h ? s->q_stride_b / s->q_stride_h : 1;
    const uint32_t k_heads = s->k_stride_b / s->k_stride_h ? s->k_stride_b / s->k_stride_h : 1;
    const uint32_t group = q_heads / k_heads ? q_heads / k_heads : 1;
    if (q_heads != n_heads || n_heads % group != 0)
        return static_fail(err, err_len, MF_ERR_INVALID_SHAPE, "strides imply %llu query heads, n_heads is %llu", q_heads, n_heads);
    if (group > 16) return static_fail(err, err_len, MF_ERR_OPERATION_NOT_SUPPORTED, "group size %llu > 16", group);
    const uint32_t cache_heads = n_heads / group;
    if (s->k_stride_h % D || s->k_stride_b % D || s->v_stride_h % D || s->v_stride_b % D)
        return static_fail(err, err_len, MF_ERR_INVALID_SHAPE, "K/V strides must be multiples of head_dim");
    if ((uint64_t)sp->kv_len * D > s->k_stride_h || (uint64_t)sp->kv_len * D > s->v_stride_h)
        return static_fail(err, err_len, MF_ERR_INVALID_OPERATION, "kv_len %llu exceeds the cache capacity", sp->kv_len);
    if ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15u)
        return static_fail(err, err_len, MF_ERR_INVALID_SHAPE, "K/V base pointers must be 16-byte aligned");

    // Same span rule as mf_flash_decode with n_splits = 0 on a context with default options, so both
    // produce the same bits (a context whose MF_OPTION_DECODE_STAGES selects another variant cuts differently).
    const uint32_t T = (sp->kv_len + kTileKeys - 1) / kTileKeys;
    const uint64_t U = (uint64_t)batch * cache_heads;
    const uint64_t total = U * T;
    if (total > 0xFFFFFFFFull) return static_fail(err, err_len, MF_ERR_OPERATION_NOT_SUPPORTED, "too many tiles");
    const uint32_t want = decode_cta_target((uint32_t)dst.sm_count, group > 8 ? 1 : 2, total);  // as mf_flash_decode
    const UniformSplit split = uniform_split((uint32_t)U, T, 0, want);
    const uint32_t span = split.span, n_ctas = split.n_ctas;
    const uint32_t HP = 8 * ((group + 7) / 8);
    const uint64_t slots = U + n_ctas;
    const uint64_t need = (uint64_t)kStaticStatusBytes + kStaticTicketBytes + slots * HP * (D + 2) * 4;
    if (U * 4 > kStaticTicketBytes || need > kStaticScratchBytes)
        return static_fail(err, err_len, MF_ERR_OUT_OF_MEMORY,
                           "this decode needs %llu bytes of scratch; the built-in array holds %llu (and 4096 batch x kv-head "
                           "units): use mf_flash_decode, which allocates",
                           need, (unsigned long long)kStaticScratchBytes);

    unsigned char *base = dst.scratch;
    if (cudaMemsetAsync(base, 0, kStaticStatusBytes + kStaticTicketBytes, stream) != cudaSuccess)
        return static_fail(err, err_len, MF_ERR_CUDA, "cudaMemsetAsync(static scratch) failed");

    DecodeParams p{};
    p.q = static_cast<const __half *>(q);
    p.out = static_cast<__half *>(output);
    p.k_base = const_cast<__half *>(static_cast<const __half *>(k));
    p.v_base = const_cast<__half *>(static_cast<const __half *>(v));
    p.status = reinterpret_cast<uint32_t *>(base);
    p.counters = reinterpret_cast<uint32_t *>(base + kStaticStatusBytes);
    p.part_acc = reinterpret_cast<float *>(base + kStaticStatusBytes + kStaticTicketBytes);
    p.part_ml = p.part_acc + slots * HP * D;
    p.n_heads = n_heads;
    p.n_kv_heads = cache_heads;
    p.group = group;
    p.batch = batch;
    p.k_rows_b = s->k_stride_b / D;
    p.k_rows_h = s->k_stride_h / D;
    p.v_rows_b = s->v_stride_b / D;
    p.v_rows_h = s->v_stride_h / D;
    p.uniform_kv_len = sp->kv_len;
    p.uniform_tiles = T;
    p.uniform_span = span;
    p.uniform_parts = split.parts;
    p.uniform_total = split.parts ? n_ctas * span : (uint32_t)total;  // the cursor turns flat / span into the CTA index
    p.q_stride_b = s->q_stride_b;
    p.q_stride_h = s->q_stride_h;
    p.out_stride_b = s->out_stride_b;
    p.out_stride_h = s->out_stride_h;
    p.scale_log2 = sp->scale * 1.4426950408889634f;
    p.rope_mode = MF_ROPE_MODE_NEOX;

    const uint64_t k_rows = (uint64_t)(batch - 1) * p.k_rows_b + (uint64_t)cache_heads * p.k_rows_h;
    const uint64_t v_rows = (uint64_t)(batch - 1) * p.v_rows_b + (uint64_t)cache_heads * p.v_rows_h;
    CUtensorMap tm_k, tm_v;
    if (!static_encode(dst, k, k_rows, D, &tm_k) || !static_encode(dst, v, v_rows, D, &tm_v))
        return static_fail(err, err_len, MF_ERR_CUDA, "cuTensorMapEncodeTiled failed");
    const uint32_t nt = (group + 7) / 8;
    cudaError_t e;
    if (D == 128)
        e = nt == 1 ? static_launch<128, 1, 3, 2>(tm_k, tm_v, p, n_ctas, stream) : static_launch<128, 2, 5, 1>(tm_k, tm_v, p, n_ctas, stream);
    else
        e = nt == 1 ? static_launch<64, 1, 6, 2>(tm_k, tm_v, p, n_ctas, stream) : static_launch<64, 2, 8, 1>(tm_k, tm_v, p, n_ctas, stream);
    if (e != cudaSuccess) return static_fail(err, err_len, MF_ERR_CUDA, "decode launch failed (%llu)", (unsigned long long)e);
    return MF_OK;
}

// Reads the status word of the built-in array without allocating: one 4-byte asynchronous copy on the
// caller's stream into the caller's (preferably pinned) host word.  Non-zero after the stream has
// drained means a device-side wait of the last mf_flash_decode_static_scratch call on this GPU ran
// out and its output is not valid.
extern "C" mf_status mf_static_scratch_status(void *cuda_stream, uint32_t *host_status)
{
    using namespace mf;
    if (!host_status) return MF_ERR_INPUT_NOT_FOUND;
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return MF_ERR_CUDA;
    if (!g_static_state[device].ready) {
        const mf_status st = static_setup(device, nullptr, 0);
        if (st != MF_OK) return st;
    }
    return cudaMemcpyAsync(host_status, g_static_state[device].scratch, 4, cudaMemcpyDeviceToHost,
                           static_cast<cudaStream_t>(cuda_stream)) == cudaSuccess ? MF_OK : MF_ERR_CUDA;
}
