// GQA flash-decode over a PAGED 8-bit (FP8 E4M3) K/V cache for sm_100a, with the append of the step's
// new token (RoPE of k, per-row quantisation) and the RoPE of q fused in.
//
// No counterpart in the reference, which only has a roadmap for a quantised cache
// (docs/FLASH.md:121-186, docs/SAGE.md:1-60).  The attention contract is the reference's
// (flash_decode.metal:146-490: q rounded to f16 after RoPE, products accumulated in f32, scores times
// `scale`, running max from -1e30, non-finite scores count as -1e30, acc / l, one rounding to f16)
// with K := the decoded bytes times the row's scale and V := the dequantised rows.
//
// Cache format (defined by this project): byte pools for K and for V, each byte an OCP FP8 E4M3 value, and scale
// pools [n_pages, Hkv, P] f32, one scale per cached row:
//     amax = max |x_i| over the row (K after RoPE and f16 rounding, V as given),
//     scale = amax / 448 (1 for an all-zero row), byte_i = e4m3_rne_satfinite(x_i / scale).
// K rows lie row-major, [n_pages, Hkv, P, 128]; V lies dim-major in blocks of 16 keys inside each (page, kv head)
// run, [n_pages, Hkv, P / 16, 128, 16] (v_off8 below).  Half the bytes of the f16 cache cross HBM per key.
//
// Kernel shape: that of decode_kernel (decode.cu) - TMA producers filling a ring of 64-key K/V tiles, four consumer
// warps on mma.sync with the query group on the 8-wide N side, consecutive tiles per CTA from the host's plan,
// partials and an atomic ticket for units cut into several spans.  What differs:
//  * a tile row is 128 bytes: one TMA box per page and tensor (K with the 128-byte swizzle, V's blocks as they lie),
//    and the page's row scales by an untiled bulk copy counted on the same mbarrier; K and V have a producer warp
//    each, which read the page table 32 ids at a time, a chunk ahead of the tiles that use them;
//  * a tile is worked on by TWO warps, 32 keys each, while the other two take the next tile: per key the softmax
//    bookkeeping (maxima by redux.sync, rescale skipped by a vote when no maximum moved) is amortised over twice the
//    keys, and the accumulators are rescaled half as often;
//  * sm_100a's legacy tensor path has no 8-bit product (ptxas expands mma.sync ... e4m3 into conversions, f16 MMAs and
//    f32 adds, measured: 2 HMMA + 4 FADD + up to 12 F2FP per instruction), so the bytes are converted here, two per
//    cvt.rn.f16x2.e4m3x2 (exact), straight from the registers ldmatrix delivers, and meet f16 MMAs whose k order is
//    permuted to match: a thread's four K bytes are dims 4c .. 4c + 3 of a 16-dim chunk (q's fragment is loaded in the
//    same order), its four V bytes keys 4c .. 4c + 3 of a 16-key block (the score MMA's rows are laid out so that the
//    transposed weights arrive in that order).  Nothing is permuted or transposed in registers;
//  * K's row scale multiplies the f32 score; V's row scale multiplies the softmax weight of its key, relative to
//    sigma, a recent maximum of the scales (so the f16 weight stays in normal range), and the accumulator is kept in
//    units of sigma, switched inside the online-softmax rescale.
#include <cuda_fp8.h>

#include <type_traits>

#include "internal.hpp"
#include "ptx.cuh"
#include "push.cuh"

namespace mf {
namespace {

constexpr uint32_t kD = 128;
constexpr uint32_t kHP = 8;  // heads per group, padded
constexpr uint32_t kStages = 6;
constexpr uint32_t kConsumerWarps = 4;
constexpr uint32_t kConsumerThreads = kConsumerWarps * 32;
constexpr uint32_t kProducerWarps = 2;  // one streams K and its scales, the other V and its scales
constexpr uint32_t kThreads = kConsumerThreads + 32 * kProducerWarps;
constexpr float kNegSentinel = -1e30f;
constexpr float kMaxSlack = 8.f;  // log2: how far a score may exceed the running reference before it moves
constexpr uint64_t kWaitLimitNs = 2000000000ull;
constexpr float kLn2 = 0.6931471805599453f;

constexpr uint32_t kTileBytes = kTileKeys * kD;  // one K or V tile: 8 KB
constexpr uint32_t kStageBytes = 2 * kTileBytes;
constexpr uint32_t kScaleStage = 2 * kTileKeys * 4;  // K scales then V scales of a tile
constexpr uint32_t kOffScales = kStages * kStageBytes;
constexpr uint32_t kCombStride = kD / 2 + 4;
constexpr uint32_t kOffComb = kOffScales + kStages * kScaleStage;
constexpr uint32_t kCombBytes = kConsumerWarps * kHP * kCombStride * 4;
constexpr uint32_t kQStride = kD + 8;       // f16 elements per head row of q (the pad spreads the heads over the banks)
constexpr uint32_t kOffQ = kOffComb + kCombBytes;
constexpr uint32_t kOffMl = kOffQ + kHP * kQStride * 2;
constexpr uint32_t kOffRow = kOffMl + kConsumerWarps * kHP * 2 * 4;  // the new k and v rows (f16) while they are quantised
constexpr uint32_t kOffRed = kOffRow + 2 * kD * 2;                  // per-warp maxima
constexpr uint32_t kOffBar = kOffRed + 2 * kConsumerWarps * 4;
constexpr uint32_t kOffFlags = kOffBar + 2 * kStages * 8;
constexpr uint32_t kTotal = kOffFlags + 16;
constexpr uint32_t kDynamic = kTotal + 1024;
static_assert(2 * (kDynamic + 1024) <= 228 * 1024, "two CTAs per SM");

struct Kv8Params {
    DecodeParams d;          // the fields shared with decode_kernel (k_base / v_base are the byte pools)
    float *k_scales, *v_scales;
};

// Byte offset of (row, 16-byte chunk) in a tile of 128-byte rows made of TMA boxes of 2^rpb_log2 rows
// (a multiple of 8, so a box is a whole number of 1 KB swizzle atoms).
__device__ __forceinline__ uint32_t tile_off8(uint32_t row, uint32_t c16)
{
    return (row << 7) + (((c16 & 7) ^ (row & 7)) << 4);
}

// V is stored dim-major in blocks of 16 keys: byte (key r, dim d) of a run of rows (a page of one kv head in the
// pool, a tile in shared memory) sits at (r / 16) * 2048 + d * 16 + r % 16.
__host__ __device__ __forceinline__ uint32_t v_off8(uint32_t r, uint32_t d)
{
    return (r >> 4) * (16u * kD) + d * 16u + (r & 15u);
}

// The low / high two E4M3 bytes of a register as f16x2 (exact: every E4M3 value is an f16 value).  The legacy
// tensor path of sm_100a has no 8-bit product - ptxas expands mma.sync ... e4m3 into these conversions, f16 MMAs
// and an f32 add per accumulator register - so the conversions are written out and counted here.
__device__ __forceinline__ uint32_t e4m3x2_lo_to_f16x2(uint32_t r)
{
    uint32_t d;
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, lo;\n\t}" : "=r"(d) : "r"(r));
    return d;
}
__device__ __forceinline__ uint32_t e4m3x2_hi_to_f16x2(uint32_t r)
{
    uint32_t d;
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, hi;\n\t}" : "=r"(d) : "r"(r));
    return d;
}
// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col); a pure function of its registers (not volatile), so that
// the compiler may move it among the conversions
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Untiled bulk copy global -> shared (both addresses 16-byte aligned, size a multiple of 16); completion is
// counted on `bar` as transaction bytes, like a tile copy.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void rope_pair(float xi, float xj, float c, float s, __half &oi, __half &oj)
{
    oi = __float2half_rn(__fsub_rn(__fmul_rn(xi, c), __fmul_rn(xj, s)));
    oj = __float2half_rn(__fadd_rn(__fmul_rn(xj, c), __fmul_rn(xi, s)));
}

// PUSH: the sequence-sharded forms that hand the partials to the other ranks themselves (a separate instantiation, so
// that the plain form carries none of that code: merely present, it cost the batched step 7 %).
// Item i of the plan; in the cluster form (CL) item i belongs to cluster i and this CTA takes an equal share of its
// tiles (the first `rem` CTAs one more).
template <bool CL>
__device__ __forceinline__ WorkItem load_item(const DecodeParams &p, uint32_t i)
{
    WorkItem it = p.items[i];
    if (CL) {
        const uint32_t C = p.cluster_size, r = cluster_cta_rank();
        const uint32_t tiles = it.tile_end - it.tile_begin, base = tiles / C, rem = tiles - base * C;
        it.tile_begin += r * base + min(r, rem);
        it.tile_end = it.tile_begin + base + (r < rem ? 1u : 0u);
    }
    return it;
}

// CL: the cluster form of decode_kernel (decode.cu) - the CTAs of a unit (or of one range of it) form a thread-block
// cluster, every CTA owns head_dim / C dims of every head, the CTAs' combined accumulators meet in the owners' shared
// memory (in the area the plain form's combine uses: nothing else touches it while tiles stream) and one cluster
// barrier later every owner reduces its columns.  A separate instantiation, like PUSH.
template <bool PUSH, bool CL>
__global__ void __launch_bounds__(kThreads, 2)
decode_kv8_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const Kv8Params kp)
{
    const DecodeParams &p = kp.d;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t bar_full = smem_base + kOffBar, bar_empty = bar_full + kStages * 8;
    volatile uint32_t *flags = reinterpret_cast<volatile uint32_t *>(smem + kOffFlags);

    if (tid == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            mbar_init(bar_full + s * 8, kProducerWarps);  // each producer warp's expect-tx arrival
            mbar_init(bar_empty + s * 8, 2);  // the two warps that work on the tile
        }
        flags[0] = 0;
        flags[1] = 0;
        mbar_fence_init();
        fence_proxy_async();
    }
    __syncthreads();

    const uint32_t P = p.page_size;  // a power of two in 8..64
    const uint32_t boxes_per_tile = kTileKeys / P;
    // (cluster form: dependents are released when the V producer has requested its last tile, as in decode_kernel)
    if (!p.strict_release && !p.release_late) grid_launch_dependents();

    if (warp >= kConsumerWarps) {
        // ------------------------------------------------------- two producer warps ---
        // With 2 KB per TMA box (a 16-row page of one kv head) the issue rate of the copies, not their bytes,
        // limits a producer: K and V are streamed by a warp each.
        const bool is_v = warp > kConsumerWarps;
        const CUtensorMap *tm = is_v ? &tm_v : &tm_k;
        const float *scales = is_v ? kp.v_scales : kp.k_scales;
        if (lane == 0) tma_prefetch_desc(tm);
        if (!p.early_stream) grid_dependency_wait();
        const uint64_t policy = l2_policy_evict_first();
        uint32_t idx = CL ? blockIdx.x / p.cluster_size : p.cta_item_begin[blockIdx.x];
        const uint32_t end = CL ? idx + 1 : p.cta_item_begin[blockIdx.x + 1];
        uint32_t stage = 0, phase = 0, issued = 0;
        // Page ids travel 32 at a time, one per lane, a chunk ahead of the tiles that use them: a lookup per tile in
        // front of its copies had put one global-load latency into every tile of the stream.  The same goes for the
        // items: the next item, its length and its first ids are fetched while this item's tiles are issued.
        auto ids_of = [&](const WorkItem &w, uint32_t len, uint32_t base) -> uint32_t {
            return base + lane < (len + P - 1) / P ? __ldg(p.page_table + (size_t)w.seq * p.pt_stride + base + lane) : 0u;
        };
        WorkItem it_next{};
        uint32_t L_next = 0, ids_a = 0, ids_b = 0;
        auto fetch_item = [&](uint32_t i) {
            it_next = load_item<CL>(p, i);
            L_next = min(p.kv_lens[it_next.seq], p.pt_stride * P);  // never past the page table
            ids_a = ids_of(it_next, L_next, it_next.tile_begin * boxes_per_tile);
            ids_b = ids_of(it_next, L_next, it_next.tile_begin * boxes_per_tile + 32);
        };
        if (idx < end) fetch_item(idx);
        for (; idx < end; ++idx) {
            const WorkItem it = it_next;
            const uint32_t L = L_next;
            uint32_t chunk = it.tile_begin * boxes_per_tile;
            auto load_ids = [&](uint32_t base) -> uint32_t { return ids_of(it, L, base); };
            uint32_t ids = ids_a, ids_next = ids_b;
            if (idx + 1 < end) fetch_item(idx + 1);
            for (uint32_t t = it.tile_begin; t < it.tile_end; ++t) {
                const uint32_t pg0 = t * boxes_per_tile;
                if (pg0 >= chunk + 32) {
                    ids = ids_next;
                    chunk += 32;
                    ids_next = load_ids(chunk + 32);
                }
                const uint32_t tok_box = t * kTileKeys + lane * P;
                const uint32_t page_box = __shfl_sync(0xffffffffu, ids, (pg0 - chunk + lane) & 31u);
                // The tensor map would clip a tile copy of a page outside the pool; the page's row scales come by an
                // untiled copy that nothing clips, so such a page is not fetched at all and the launch reports it.
                const bool valid = lane < boxes_per_tile && tok_box < L && page_box < p.n_pages;
                const uint32_t row_box = valid ? (page_box * p.n_kv_heads + it.kvh) * P : 0u;
                if (!valid && lane < boxes_per_tile && tok_box < L && !is_v) atomicOr(p.status, kStatusBadPage);
                if (!flags[0] && !mbar_wait_bounded(bar_empty + stage * 8, phase ^ 1, kWaitLimitNs)) {
                    flags[0] = 1;
                    atomicOr(p.status, 1u);
                }
                const uint32_t n_valid = __popc(__ballot_sync(0xffffffffu, valid));
                const uint32_t full = bar_full + stage * 8;
                if (lane == 0) mbar_arrive_expect_tx(full, n_valid * P * (kD + 4));
                __syncwarp();
                if (valid) {
                    tma_load_2d_hint(smem_base + stage * kStageBytes + (is_v ? kTileBytes : 0u) + lane * P * kD, tm, 0, (int32_t)row_box, full, policy);
                    bulk_load_1d(smem_base + kOffScales + stage * kScaleStage + (is_v ? kTileKeys * 4 : 0u) + lane * P * 4, scales + row_box, P * 4, full);
                }
                ++issued;
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
        if (p.release_late && is_v) grid_launch_dependents();
        if (flags[0]) {  // after an abort nobody waits for the ring: let our own copies land before the CTA ends
            const uint32_t n = issued < kStages ? issued : kStages;
            for (uint32_t i = 0; i < n; ++i) {
                const uint32_t s = (stage + kStages - 1 - i) % kStages;
                const uint32_t ph = (s < stage) ? phase : (phase ^ 1);
                (void)mbar_wait_bounded(bar_full + s * 8, ph, kWaitLimitNs);
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumers ---
    grid_dependency_wait();
    if (p.strict_release) grid_launch_dependents();
    if (PUSH && p.push_wait_mask) push::push_wait_for_mergers(p, tid);
    float *comb = reinterpret_cast<float *>(smem + kOffComb);
    __half *q_s = reinterpret_cast<__half *>(smem + kOffQ);  // [head][kQStride] f16
    float *ml_s = reinterpret_cast<float *>(smem + kOffMl);
    __half *row_s = reinterpret_cast<__half *>(smem + kOffRow);
    float *red_s = reinterpret_cast<float *>(smem + kOffRed);
    const uint32_t G = p.group, half_d = kD / 2;
    const uint32_t g = lane >> 2, c = lane & 3;
    const uint32_t half = warp & 1u, pair = warp >> 1;  // which 32 keys of a tile, and which tiles
    // ldmatrix row addresses of this lane (matrix lane / 8, row lane % 8).  K: MMA row i of a 16-key block is key
    // 4(i/2) + i%2, row i + 8 that key + 2 (the order in which the transposed weights meet V's bytes); the two right-hand
    // matrices are the next 16 dims.  V: rows are dims, 32 of them per load, 16 keys wide.
    const uint32_t k_row = 32 * half + 4 * ((lane & 7) >> 1) + (lane & 1) + 2 * ((lane >> 3) & 1);
    const uint32_t koff = k_row * kD, ksw = ((lane >> 4) ^ (k_row & 7)) << 4;
    const uint32_t voff = half * (32 * kD) + lane * 16;
    const uint32_t key_lo = 4 * (g >> 1) + (g & 1);  // key (within a block) of accumulator rows g | g + 8: key_lo | key_lo + 2

    uint32_t idx = CL ? blockIdx.x / p.cluster_size : p.cta_item_begin[blockIdx.x];
    const uint32_t end = CL ? idx + 1 : p.cta_item_begin[blockIdx.x + 1];
    uint32_t stage = 0, phase = 0;
    // The next item and its length are fetched while this item's tiles stream: two dependent loads less between
    // the last tile of one item and the first of the next (what an item costs is what the step planner charges).
    WorkItem it_next{};
    uint32_t L_next = 0, pos_next = 0;
    if (idx < end) {
        it_next = load_item<CL>(p, idx);
        L_next = p.kv_lens[it_next.seq];
        pos_next = p.rope_positions ? p.rope_positions[it_next.seq] : 0u;
    }
    for (; idx < end; ++idx) {
        const WorkItem it = it_next;
        const uint32_t L_dev = L_next, pos_dev = pos_next;
        if (idx + 1 < end) {
            it_next = load_item<CL>(p, idx + 1);
            L_next = p.kv_lens[it_next.seq];
            pos_next = p.rope_positions ? p.rope_positions[it_next.seq] : 0u;
        }
        const uint32_t L = min(L_dev, p.pt_stride * P);
        if (L_dev != L && tid == 0) atomicOr(p.status, kStatusBadPage);  // a length the page table has no entries for
        const uint32_t n_tiles = (L + kTileKeys - 1) / kTileKeys;
        const uint32_t pos = p.rope_positions ? pos_dev : (L ? L - 1 : 0);
        const __half *cos_row = p.cos_t + (size_t)pos * half_d, *sin_row = p.sin_t + (size_t)pos * half_d;

        // ---- q (optionally roped, rounded to f16) -> shared memory --------------------------------------
        // Every global load of this prologue is issued before the first one is used: q of the group's heads, the
        // position's cos / sin pair, and - in the CTA that will meet the sequence's last tile - the new k and v
        // row and the id of the page they go to.
        named_bar_sync(1, kConsumerThreads);
        constexpr uint32_t kQPasses = (kHP * (kD / 2)) / kConsumerThreads;
        static_assert((kHP * (kD / 2)) % kConsumerThreads == 0 && kConsumerThreads % (kD / 2) == 0, "q staging");
        const uint32_t pr = tid % half_d;  // the same pair of dims in every pass
        const uint32_t di = p.rope_mode == MF_ROPE_MODE_NORMAL ? 2 * pr : pr;
        const uint32_t dj = p.rope_mode == MF_ROPE_MODE_NORMAL ? di + 1 : pr + half_d;
        __half qi[kQPasses], qj[kQPasses];
#pragma unroll
        for (uint32_t j = 0; j < kQPasses; ++j) {
            const uint32_t hg = (tid + j * kConsumerThreads) / half_d;
            qi[j] = qj[j] = __float2half_rn(0.f);
            if (hg < G) {
                const __half *src = p.q + (size_t)it.seq * p.q_stride_b + (size_t)(it.kvh * G + hg) * p.q_stride_h;
                qi[j] = src[di];
                qj[j] = src[dj];
            }
        }
        float cs = 1.f, sn = 0.f;
        if (p.rope) {
            cs = __half2float(cos_row[pr]);
            sn = __half2float(sin_row[pr]);
        }
        const bool ends_seq = p.append && it.tile_begin < n_tiles && it.tile_end >= n_tiles;
        __half kn_i = __float2half_rn(0.f), kn_j = kn_i, vn = kn_i;
        uint32_t new_page = 0;
        if (ends_seq) {
            if (tid < half_d) {
                const __half *ks = p.k_new + (size_t)it.seq * p.knew_stride_b + (size_t)it.kvh * kD;
                kn_i = ks[di];
                kn_j = ks[dj];
            }
            vn = p.v_new[(size_t)it.seq * p.knew_stride_b + (size_t)it.kvh * kD + tid];
            new_page = p.page_table[(size_t)it.seq * p.pt_stride + (L - 1) / P];
        }
#pragma unroll
        for (uint32_t j = 0; j < kQPasses; ++j) {
            const uint32_t hg = (tid + j * kConsumerThreads) / half_d;
            __half oi = qi[j], oj = qj[j];
            if (hg < G) {
                if (p.rope) rope_pair(__half2float(oi), __half2float(oj), cs, sn, oi, oj);
                if (p.q_rot && it.tile_begin == 0) {
                    __half *dst = p.q_rot + (size_t)it.seq * p.q_stride_b + (size_t)(it.kvh * G + hg) * p.q_stride_h;
                    dst[di] = oi;
                    dst[dj] = oj;
                }
            }
            q_s[hg * kQStride + di] = oi;
            q_s[hg * kQStride + dj] = oj;
        }
        if (ends_seq && p.rope) rope_pair(__half2float(kn_i), __half2float(kn_j), cs, sn, kn_i, kn_j);
        named_bar_sync(1, kConsumerThreads);
        // B fragments of Q^T (k = 16 dims x n = 8 heads per step).  A thread's four K bytes are dims 4c .. 4c + 3 of the
        // 16-dim chunk, so MMA k-index 2c, 2c + 1 stands for dims 4c, 4c + 1 and 2c + 8, 2c + 9 for dims 4c + 2, 4c + 3.
        uint32_t bq[kD / 16][2];
#pragma unroll
        for (int ks = 0; ks < (int)kD / 16; ++ks) {
            const uint2 w = *reinterpret_cast<const uint2 *>(q_s + g * kQStride + 16 * ks + 4 * c);
            bq[ks][0] = w.x;
            bq[ks][1] = w.y;
        }
        float m_run[2] = {kNegSentinel, kNegSentinel}, l_run[2] = {0.f, 0.f};  // l: this thread's keys only, summed at the end
        float sigma = 0.f, wsc = 0.f;  // the accumulators are in units of sigma (a V row scale); wsc = 1 / sigma
        float o[kD / 16][4];
#pragma unroll
        for (int mt = 0; mt < (int)kD / 16; ++mt) o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f;

        for (uint32_t t = it.tile_begin; t < it.tile_end; ++t) {
            // A tile is worked on by two warps, 32 keys each; the other two take the next tile.  The tile that holds
            // position L - 1 is first patched by all four.
            const bool mine = ((t - it.tile_begin) & 1u) == pair, last = t + 1 == n_tiles;
            if ((mine || last) && !flags[0] && !mbar_wait_bounded(bar_full + stage * 8, phase, kWaitLimitNs)) {
                flags[0] = 1;
                atomicOr(p.status, 2u);
            }
            uint8_t *k_tile = smem + stage * kStageBytes, *v_tile = k_tile + kTileBytes;
            const uint32_t k_addr = smem_base + stage * kStageBytes, v_addr = k_addr + kTileBytes;
            float *ksc = reinterpret_cast<float *>(smem + kOffScales + stage * kScaleStage), *vsc = ksc + kTileKeys;
            const uint32_t key0 = t * kTileKeys;
            if (last) {
                // The tile that holds position L - 1: quantise and splice in the token appended by this step (and
                // store it to the cache), then neutralise the rows past L (stale bytes, stale or NaN scales).
                const uint32_t r_new = (L - 1) - key0;
                bool store_ok = p.append != 0;
                uint32_t new_row = 0;
                if (p.append) {
                    const uint32_t page = new_page;  // read in the prologue
                    store_ok = page < p.n_pages;
                    if (!store_ok && tid == 0) atomicOr(p.status, kStatusBadPage);
                    new_row = (page * p.n_kv_heads + it.kvh) * P + (L - 1) % P;
                }
                if (store_ok) {
                    if (tid < half_d) {  // the pair this thread roped in the prologue
                        row_s[di] = kn_i;
                        row_s[dj] = kn_j;
                    }
                    row_s[kD + tid] = vn;
                    named_bar_sync(2, kConsumerThreads);
                    // one element of each row per thread: row maxima by warp shuffles and four words of shared memory
                    const float xk = __half2float(row_s[tid]), xv = __half2float(row_s[kD + tid]);
                    float ak = fabsf(xk), av = fabsf(xv);
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) {
                        ak = fmaxf(ak, __shfl_xor_sync(0xffffffffu, ak, off));
                        av = fmaxf(av, __shfl_xor_sync(0xffffffffu, av, off));
                    }
                    if (lane == 0) {
                        red_s[warp] = ak;
                        red_s[kConsumerWarps + warp] = av;
                    }
                    named_bar_sync(2, kConsumerThreads);
                    const float amax_k = fmaxf(fmaxf(red_s[0], red_s[1]), fmaxf(red_s[2], red_s[3]));
                    const float amax_v = fmaxf(fmaxf(red_s[4], red_s[5]), fmaxf(red_s[6], red_s[7]));
                    const float sk = amax_k > 0.f ? __fdiv_rn(amax_k, 448.f) : 1.f, sv = amax_v > 0.f ? __fdiv_rn(amax_v, 448.f) : 1.f;
                    const uint8_t qk = (uint8_t)__nv_cvt_float_to_fp8(__fdiv_rn(xk, sk), __NV_SATFINITE, __NV_E4M3);
                    const uint8_t qv = (uint8_t)__nv_cvt_float_to_fp8(__fdiv_rn(xv, sv), __NV_SATFINITE, __NV_E4M3);
                    reinterpret_cast<uint8_t *>(p.k_base)[(size_t)new_row * kD + tid] = qk;
                    reinterpret_cast<uint8_t *>(p.v_base)[(size_t)(new_row - (L - 1) % P) * kD + v_off8((L - 1) % P, tid)] = qv;
                    k_tile[tile_off8(r_new, tid >> 4) + (tid & 15)] = qk;
                    v_tile[v_off8(r_new, tid)] = qv;
                    if (tid == 0) {
                        kp.k_scales[new_row] = sk;
                        kp.v_scales[new_row] = sv;
                        ksc[r_new] = sk;
                        vsc[r_new] = sv;
                    }
                }
                const uint32_t first_dead = L - key0;  // 1..64
                for (uint32_t r = first_dead + tid; r < kTileKeys; r += kConsumerThreads) vsc[r] = 0.f;
                // stale bytes of V past L could decode to NaN, and 0 * NaN is NaN: clear them, 16 keys of a dim at a time
                for (uint32_t ch = (first_dead >> 4) * kD + tid; ch < (kTileKeys / 16) * kD; ch += kConsumerThreads) {
                    const uint32_t blk = ch / kD, keep = first_dead > blk * 16 ? first_dead - blk * 16 : 0u;  // < 16 only in the first block touched
                    uint4 *w = reinterpret_cast<uint4 *>(v_tile + ch * 16);
                    if (keep == 0) {
                        *w = make_uint4(0, 0, 0, 0);
                    } else if (keep < 16) {
                        uint4 x = *w;
                        uint32_t *xw = reinterpret_cast<uint32_t *>(&x);
#pragma unroll
                        for (uint32_t i = 0; i < 4; ++i) {
                            const uint32_t lo = 4 * i;
                            const uint32_t m = keep >= lo + 4 ? 0xFFFFFFFFu : (keep > lo ? (1u << (8 * (keep - lo))) - 1u : 0u);
                            xw[i] &= m;
                        }
                        *w = x;
                    }
                }
                fence_proxy_async();
                named_bar_sync(2, kConsumerThreads);
            }


            const uint32_t ukey0 = key0 + 32 * half;
            if (mine && ukey0 < L) {
                // ---- S^T (2 x 16 keys x 8 heads) = K_tile Q^T: bytes -> f16 in registers, f16 MMAs, four accumulator
                //      chains in rotation ----------------------------------------------------------------------------
                float acc[2][2][4];  // [16-key block][even | odd 16-dim step]
#pragma unroll
                for (int b = 0; b < 2; ++b)
#pragma unroll
                    for (int kk = 0; kk < 2; ++kk) acc[b][kk][0] = acc[b][kk][1] = acc[b][kk][2] = acc[b][kk][3] = 0.f;
#pragma unroll
                for (int kq = 0; kq < (int)kD / 32; ++kq) {
                    uint32_t r[2][4];
#pragma unroll
                    for (int b = 0; b < 2; ++b)
                        // four 8 x 16-byte matrices: (rows 0-7 | rows 8-15) x (dims 32kq .. +15 | +16 .. +31)
                        ldmatrix_x4(r[b], k_addr + koff + b * (16 * kD) + (ksw ^ (kq * 32)));
#pragma unroll
                    for (int b = 0; b < 2; ++b) {
                        mma_f16(acc[b][0], e4m3x2_lo_to_f16x2(r[b][0]), e4m3x2_lo_to_f16x2(r[b][1]), e4m3x2_hi_to_f16x2(r[b][0]),
                                e4m3x2_hi_to_f16x2(r[b][1]), bq[2 * kq][0], bq[2 * kq][1]);
                        mma_f16(acc[b][1], e4m3x2_lo_to_f16x2(r[b][2]), e4m3x2_lo_to_f16x2(r[b][3]), e4m3x2_hi_to_f16x2(r[b][2]),
                                e4m3x2_hi_to_f16x2(r[b][3]), bq[2 * kq + 1][0], bq[2 * kq + 1][1]);
                    }
                }
                // ---- the rows' scales; scores in the log2 domain --------------------------------------------------
                float sc[2][4], vlo[2], vhi[2];
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    const uint32_t at = 32 * half + 16 * b + key_lo;
                    const float k_lo = ksc[at] * p.scale_log2, k_hi = ksc[at + 2] * p.scale_log2;
                    vlo[b] = vsc[at];  // rows past L were set to 0
                    vhi[b] = vsc[at + 2];
                    // non-finite scores count as -1e30: fmaxf maps NaN and -inf there; +inf shows in the maxima below
#pragma unroll
                    for (int i = 0; i < 4; ++i) sc[b][i] = fmaxf((acc[b][0][i] + acc[b][1][i]) * (i < 2 ? k_lo : k_hi), kNegSentinel);
                }
                bool dead[2][2] = {{false, false}, {false, false}};
                if (last) {
#pragma unroll
                    for (int b = 0; b < 2; ++b) {
                        const uint32_t kr = ukey0 + 16 * b + key_lo;
                        dead[b][0] = kr >= L;
                        dead[b][1] = kr + 2 >= L;
                        if (dead[b][0]) sc[b][0] = sc[b][1] = kNegSentinel;
                        if (dead[b][1]) sc[b][2] = sc[b][3] = kNegSentinel;
                    }
                }
                // ---- online softmax over the 32 keys.  The running maximum is only a reference point: it moves when a
                //      score exceeds it by more than 8 (log2), so weights stay below 2^8 and the accumulators are rescaled
                //      a few times per span instead of whenever one of eight heads sees a new record ------------------------
                float mx0 = fmaxf(fmaxf(sc[0][0], sc[0][2]), fmaxf(sc[1][0], sc[1][2]));
                float mx1 = fmaxf(fmaxf(sc[0][1], sc[0][3]), fmaxf(sc[1][1], sc[1][3]));
#pragma unroll
                for (int off = 4; off <= 16; off <<= 1) {
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
                }
                if (__any_sync(0xffffffffu, !(mx0 <= 3.0e38f) || !(mx1 <= 3.0e38f))) {  // an infinite score somewhere: once more without it
#pragma unroll
                    for (int b = 0; b < 2; ++b)
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (!(sc[b][i] <= 3.0e38f)) sc[b][i] = kNegSentinel;
                    mx0 = fmaxf(fmaxf(sc[0][0], sc[0][2]), fmaxf(sc[1][0], sc[1][2]));
                    mx1 = fmaxf(fmaxf(sc[0][1], sc[0][3]), fmaxf(sc[1][1], sc[1][3]));
#pragma unroll
                    for (int off = 4; off <= 16; off <<= 1) {
                        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
                        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
                    }
                }
                // V's row scales ride on the weights: weight * scale / sigma, sigma a recent maximum of the scales (at most
                // 8 times the largest of these 32), so that the f16 weight stays in normal range whatever the rows' magnitudes.
                float vmax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fmaxf(fmaxf(vlo[0], vhi[0]), fmaxf(vlo[1], vhi[1])))));
                if (!(vmax > 0.f)) vmax = 1.f;
                const bool keep_sigma = vmax <= sigma && vmax * 8.f >= sigma;
                const bool up0 = mx0 > m_run[0] + kMaxSlack, up1 = mx1 > m_run[1] + kMaxSlack;
                if (__any_sync(0xffffffffu, up0 || up1 || !keep_sigma)) {
                    const float mn0 = up0 ? mx0 : m_run[0], mn1 = up1 ? mx1 : m_run[1];
                    const float sig_new = keep_sigma ? sigma : vmax;
                    wsc = __frcp_rn(sig_new);
                    const float rs = sigma * wsc;
                    const float a0 = fast_exp2(m_run[0] - mn0), a1 = fast_exp2(m_run[1] - mn1);
                    const float f0o = a0 * rs, f1o = a1 * rs;
#pragma unroll
                    for (int mt = 0; mt < (int)kD / 16; ++mt) {
                        o[mt][0] *= f0o;
                        o[mt][1] *= f1o;
                        o[mt][2] *= f0o;
                        o[mt][3] *= f1o;
                    }
                    l_run[0] *= a0;
                    l_run[1] *= a1;
                    m_run[0] = mn0;
                    m_run[1] = mn1;
                    sigma = sig_new;
                }
                // ---- weights, transposed into the B fragments of the second product: (keys 4c, 4c + 1 | 4c + 2, 4c + 3) of head g ----
                uint32_t bp[2][2];
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    float pw[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) pw[i] = dead[b][i >> 1] ? 0.f : fast_exp2(sc[b][i] - m_run[i & 1]);
                    l_run[0] += pw[0] + pw[2];
                    l_run[1] += pw[1] + pw[3];
                    const float w_lo = vlo[b] * wsc, w_hi = vhi[b] * wsc;
                    bp[b][0] = movmatrix_trans(pack_f16x2(pw[0] * w_lo, pw[1] * w_lo));
                    bp[b][1] = movmatrix_trans(pack_f16x2(pw[2] * w_hi, pw[3] * w_hi));
                }
                // ---- O^T (dims x heads) += V_tile^T W: a load brings 32 dims x 16 keys of bytes as they lie in the dim-major
                //      blocks; low / high halves of a register are keys 4c, 4c + 1 | 4c + 2, 4c + 3 -----------------------
#pragma unroll
                for (int b = 0; b < 2; ++b)
#pragma unroll
                    for (int mq = 0; mq < (int)kD / 32; ++mq) {
                        uint32_t r[4];
                        ldmatrix_x4(r, v_addr + voff + b * (16 * kD) + mq * 512);
                        mma_f16(o[2 * mq], e4m3x2_lo_to_f16x2(r[0]), e4m3x2_lo_to_f16x2(r[1]), e4m3x2_hi_to_f16x2(r[0]), e4m3x2_hi_to_f16x2(r[1]),
                                bp[b][0], bp[b][1]);
                        mma_f16(o[2 * mq + 1], e4m3x2_lo_to_f16x2(r[2]), e4m3x2_lo_to_f16x2(r[3]), e4m3x2_hi_to_f16x2(r[2]),
                                e4m3x2_hi_to_f16x2(r[3]), bp[b][0], bp[b][1]);
                    }
            }
            __syncwarp();
            if (mine && lane == 0) mbar_arrive(bar_empty + stage * 8);
            if (++stage == kStages) {
                stage = 0;
                phase ^= 1;
            }
        }

        // ---- combine the four warps' states ---------------------------------------------------------------
#pragma unroll
        for (int off = 4; off <= 16; off <<= 1) {
            l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], off);
            l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], off);
        }
        if (lane < 4) {
            float *dst = ml_s + ((warp * kHP) + 2 * lane) * 2;
            dst[0] = m_run[0];
            dst[1] = l_run[0];
            dst[2] = m_run[1];
            dst[3] = l_run[1];
        }
        named_bar_sync(1, kConsumerThreads);
        float fac[2];
        {
            const uint32_t h0 = 2 * c;
            float ma0 = kNegSentinel, ma1 = kNegSentinel;
#pragma unroll
            for (uint32_t w = 0; w < kConsumerWarps; ++w) {
                ma0 = fmaxf(ma0, ml_s[(w * kHP + h0) * 2]);
                ma1 = fmaxf(ma1, ml_s[(w * kHP + h0 + 1) * 2]);
            }
            fac[0] = fast_exp2(m_run[0] - ma0) * sigma;
            fac[1] = fast_exp2(m_run[1] - ma1) * sigma;
        }
        const bool direct = it.n_parts == 1;
        const uint32_t C = CL ? p.cluster_size : 1u;
        if (CL) {
            const uint32_t crank = cluster_cta_rank(), own_dims = kD / C;  // C is a power of two up to 16
            const uint32_t recv_acc_addr = smem_base + kOffComb, recv_ml_addr = recv_acc_addr + kHP * kD * 4;
            static_assert(kHP * kD * 4 + 16 * kHP * 2 * 4 <= kCombBytes, "the receive area takes the combine area's place");
            // One item per CTA in this form, so the ring is idle by now: its first bytes take the four warps'
            // accumulators at full width, in one pass.
            constexpr uint32_t kFS = kD + 4;  // floats per head row
            float *cf = reinterpret_cast<float *>(smem);
            {
                float *c0 = cf + (warp * kHP + 2 * c) * kFS, *c1 = c0 + kFS;
#pragma unroll
                for (int mt = 0; mt < (int)kD / 16; ++mt) {
                    const uint32_t d0 = mt * 16 + g;  // accumulator rows are dims g and g + 8 of the chunk
                    c0[d0] = o[mt][0] * fac[0];
                    c1[d0] = o[mt][1] * fac[1];
                    c0[d0 + 8] = o[mt][2] * fac[0];
                    c1[d0 + 8] = o[mt][3] * fac[1];
                }
            }
            named_bar_sync(2, kConsumerThreads);
            // this CTA's (m, l) of every head to every CTA of the cluster
            for (uint32_t i2 = tid; i2 < C * kHP; i2 += kConsumerThreads) {
                const uint32_t r = i2 / kHP, hg = i2 - r * kHP;
                float m_all = kNegSentinel;
#pragma unroll
                for (uint32_t w = 0; w < kConsumerWarps; ++w) m_all = fmaxf(m_all, ml_s[(w * kHP + hg) * 2]);
                float l_all = 0.f;
#pragma unroll
                for (uint32_t w = 0; w < kConsumerWarps; ++w)
                    l_all += ml_s[(w * kHP + hg) * 2 + 1] * fast_exp2(ml_s[(w * kHP + hg) * 2] - m_all);
                st_cluster_f2(cluster_map_shared(recv_ml_addr + (crank * kHP + hg) * 8, r), m_all, l_all);
            }
            // four heads of one dim per thread: one 16-byte store into the owner's shared memory
            for (uint32_t e = tid; e < (kHP / 4) * kD; e += kConsumerThreads) {
                const uint32_t gq = e / kD, d = e - gq * kD;
                if (gq * 4 >= G) continue;  // padded heads are never read
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (uint32_t w = 0; w < kConsumerWarps; ++w) {
                    const float *c4 = cf + (w * kHP + gq * 4) * kFS + d;
                    acc.x += c4[0];
                    acc.y += c4[kFS];
                    acc.z += c4[2 * kFS];
                    acc.w += c4[3 * kFS];
                }
                const uint32_t owner = d / own_dims, dl = d - owner * own_dims;
                st_cluster_f4(cluster_map_shared(recv_acc_addr + ((crank * own_dims + dl) * kHP + gq * 4) * 4, owner), acc);
            }
            // ---- the cluster's CTAs meet: every store above has landed once all of them have arrived ----
            __syncwarp();
            cluster_arrive_release();
            cluster_wait_acquire();
            const float *racc = reinterpret_cast<const float *>(smem + kOffComb);
            const float2 *rml = reinterpret_cast<const float2 *>(smem + kOffComb + kHP * kD * 4);
            for (uint32_t col = tid; col < own_dims * kHP; col += kConsumerThreads) {  // (dim, head) columns this CTA owns
                const uint32_t hg = col % kHP, dl = col / kHP, d = crank * own_dims + dl;
                if (hg >= G) continue;
                float mx = kNegSentinel;
#pragma unroll 4
                for (uint32_t r = 0; r < C; ++r) mx = fmaxf(mx, rml[r * kHP + hg].x);
                float lt = 0.f, acc = 0.f;
#pragma unroll 4
                for (uint32_t r = 0; r < C; ++r) {
                    const float2 ml = rml[r * kHP + hg];
                    const float w = fast_exp2(ml.x - mx);
                    lt += ml.y * w;
                    acc += racc[(r * own_dims + dl) * kHP + hg] * w;
                }
                const uint32_t h = it.kvh * G + hg;
                if (!direct) {
                    // the cluster's partial of the unit; the CTA that completes the unit merges (ticket below)
                    p.part_acc[((size_t)it.slot * kHP + hg) * kD + d] = acc;
                    if (d == 0) *reinterpret_cast<float2 *>(p.part_ml + ((size_t)it.slot * kHP + hg) * 2) = make_float2(mx * kLn2, lt);
                } else if (PUSH && p.push_world) {
                    const size_t rows = (size_t)p.batch * p.n_heads, rowi = (size_t)it.seq * p.n_heads + h;
                    for (uint32_t r = 0; r < p.push_world; ++r) {
                        push::push_store(p, r, rowi * kD + d, acc);
                        if (d == 0) {
                            push::push_store(p, r, rows * kD + rowi, mx * kLn2);
                            push::push_store(p, r, rows * kD + rows + rowi, lt);
                        }
                    }
                } else if (p.out_acc) {
                    p.out_acc[((size_t)it.seq * p.n_heads + h) * kD + d] = acc;
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
                if (!PUSH || !p.push_world) continue;  // nobody reads another CTA's shared memory after the barrier: done
                // counted form: every CTA's share must be in the peers' blocks before the first CTA announces it (one
                // cumulative fence by the announcing threads, after this barrier); tagged words need neither
                if (!p.push_tagged) {
                    __syncwarp();
                    cluster_arrive_release();
                    cluster_wait_acquire();
                }
                if (crank == 0) push::push_signal_and_merge<(int)kD>(p, it, tid, flags);
                continue;
            }
            // not direct: every CTA of every cluster of the unit takes a ticket below; the last one merges
        }
#pragma unroll
        for (int hp = 0; hp < (CL ? 0 : 2); ++hp) {
            {
                float *c0 = comb + (warp * kHP + 2 * c) * kCombStride, *c1 = c0 + kCombStride;
#pragma unroll
                for (int mh = 0; mh < (int)kD / 32; ++mh) {
                    const int mt = hp * (kD / 32) + mh;
                    const uint32_t d0 = mh * 16 + g;  // accumulator rows are dims g and g + 8 of the chunk
                    c0[d0] = o[mt][0] * fac[0];
                    c1[d0] = o[mt][1] * fac[1];
                    c0[d0 + 8] = o[mt][2] * fac[0];
                    c1[d0 + 8] = o[mt][3] * fac[1];
                }
            }
            named_bar_sync(2, kConsumerThreads);
            for (uint32_t e = tid; e < kHP * (kD / 2); e += kConsumerThreads) {
                const uint32_t hg = e / (kD / 2), dd = e - hg * (kD / 2), d = hp * (kD / 2) + dd;
                float m_all = kNegSentinel;
#pragma unroll
                for (uint32_t w = 0; w < kConsumerWarps; ++w) m_all = fmaxf(m_all, ml_s[(w * kHP + hg) * 2]);
                float l_all = 0.f, acc = 0.f;
#pragma unroll
                for (uint32_t w = 0; w < kConsumerWarps; ++w) {
                    l_all += ml_s[(w * kHP + hg) * 2 + 1] * fast_exp2(ml_s[(w * kHP + hg) * 2] - m_all);
                    acc += comb[(w * kHP + hg) * kCombStride + dd];
                }
                if (!direct) {
                    p.part_acc[((size_t)it.slot * kHP + hg) * kD + d] = acc;
                    if (d == 0) {
                        p.part_ml[((size_t)it.slot * kHP + hg) * 2] = m_all * kLn2;
                        p.part_ml[((size_t)it.slot * kHP + hg) * 2 + 1] = l_all;
                    }
                } else if (hg < G) {
                    const uint32_t h = it.kvh * G + hg;
                    if (PUSH && p.push_world) {  // sequence-sharded, fused exchange: the partial goes to every rank
                        const size_t rows = (size_t)p.batch * p.n_heads, rowi = (size_t)it.seq * p.n_heads + h;
                        for (uint32_t r = 0; r < p.push_world; ++r) {
                            push::push_store(p, r, rowi * kD + d, acc);
                            if (d == 0) {
                                push::push_store(p, r, rows * kD + rowi, m_all * kLn2);
                                push::push_store(p, r, rows * kD + rows + rowi, l_all);
                            }
                        }
                    } else if (p.out_acc) {  // sequence-sharded: this shard's unnormalised partial
                        p.out_acc[((size_t)it.seq * p.n_heads + h) * kD + d] = acc;
                        if (d == 0) {
                            p.out_m[(size_t)it.seq * p.n_heads + h] = m_all * kLn2;
                            p.out_l[(size_t)it.seq * p.n_heads + h] = l_all;
                        }
                    } else {
                        const bool ok = (fabsf(l_all) <= 3.0e38f) && fabsf(l_all) > 1e-6f;
                        float r1 = ok ? acc / l_all : acc;
                        if (!(fabsf(r1) <= 3.0e38f)) r1 = 0.f;
                        p.out[(size_t)it.seq * p.out_stride_b + (size_t)h * p.out_stride_h + d] = __float2half_rn(r1);
                    }
                }
            }
            if (hp == 0) named_bar_sync(1, kConsumerThreads);
        }
        if (!CL && direct) {
            if (PUSH && p.push_world) push::push_signal_and_merge<(int)kD>(p, it, tid, flags);
            continue;
        }

        // ---- ticket: the CTA that completes the unit merges its partials (flash_prefill.metal:843-888) -------
        __threadfence();
        named_bar_sync(1, kConsumerThreads);
        if (tid == 0) {
            const uint32_t old = atomicAdd(p.counters + it.unit, 1u);
            const uint32_t last = (old + 1 == it.n_parts * C) ? 1u : 0u;  // cluster form: every CTA of the unit's clusters arrives
            if (last) p.counters[it.unit] = 0;
            flags[1] = last;
        }
        named_bar_sync(2, kConsumerThreads);
        if (!flags[1]) continue;
        __threadfence();
        // Merge (flash_prefill.metal:843-888), arranged so that the loads of one round trip are all in flight
        // together: this runs at the end of a CTA's work, where latency is not hidden.  Pass 1: the parts' (m, l)
        // over all threads (a head per eight threads), maxima cached in shared memory.
        constexpr uint32_t kMergeCap = 64;                    // parts whose m is cached in shared memory
        constexpr uint32_t kPerHead = kConsumerThreads / kHP; // threads per head in pass 1
        constexpr uint32_t kFlight = 20, kFlightFew = 8;      // partials in flight together in pass 2
        static_assert((kMergeCap * kHP + kConsumerThreads * 2) * 4 <= kConsumerWarps * kHP * kCombStride * 4, "merge scratch");
        float *msv = comb;                                    // [kMergeCap][kHP]
        float *red = comb + kMergeCap * kHP;                  // [threads][2]
        {
            const uint32_t g1 = tid % kHP;
            float m_loc = kNegSentinel, l_loc = 0.f;
            for (uint32_t sp = tid / kHP; sp < it.n_parts; sp += kPerHead) {
                const float2 ml = __ldcg(reinterpret_cast<const float2 *>(p.part_ml) + (size_t)(it.first_slot + sp) * kHP + g1);
                if (sp < kMergeCap) msv[sp * kHP + g1] = ml.x;
                const float mn = fmaxf(m_loc, ml.x);
                l_loc = l_loc * __expf(m_loc - mn) + (ml.y > 0.f ? ml.y * __expf(ml.x - mn) : 0.f);
                m_loc = mn;
            }
            red[tid * 2] = m_loc;
            red[tid * 2 + 1] = l_loc;
        }
        named_bar_sync(1, kConsumerThreads);
        // Pass 2: one float4 column of one real head per thread and round.
        for (uint32_t c4 = tid; c4 < G * (kD / 4); c4 += kConsumerThreads) {
            const uint32_t hg = c4 / (kD / 4), d0 = (c4 % (kD / 4)) * 4;
            float mx = kNegSentinel, lt = 0.f;
#pragma unroll
            for (uint32_t j = 0; j < kPerHead; ++j) mx = fmaxf(mx, red[(j * kHP + hg) * 2]);
#pragma unroll
            for (uint32_t j = 0; j < kPerHead; ++j) lt += red[(j * kHP + hg) * 2 + 1] * __expf(red[(j * kHP + hg) * 2] - mx);
            auto accumulate = [&](auto flight) {
                constexpr uint32_t F = decltype(flight)::value;
                float4 a4 = make_float4(0.f, 0.f, 0.f, 0.f);
                for (uint32_t s0 = 0; s0 < it.n_parts; s0 += F) {
                    float4 v[F];
                    float w[F];
#pragma unroll
                    for (uint32_t j = 0; j < F; ++j) {
                        const uint32_t sp = s0 + j;
                        if (sp < it.n_parts) {
                            const size_t sl = it.first_slot + sp;
                            v[j] = __ldcg(reinterpret_cast<const float4 *>(p.part_acc + (sl * kHP + hg) * kD + d0));
                            const float ms = sp < kMergeCap ? msv[sp * kHP + hg] : __ldcg(p.part_ml + (sl * kHP + hg) * 2);
                            w[j] = __expf(ms - mx);
                        } else {
                            v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                            w[j] = 0.f;
                        }
                    }
#pragma unroll
                    for (uint32_t j = 0; j < F; ++j) {
                        a4.x += v[j].x * w[j];
                        a4.y += v[j].y * w[j];
                        a4.z += v[j].z * w[j];
                        a4.w += v[j].w * w[j];
                    }
                }
                return a4;
            };
            const float4 acc = it.n_parts <= kFlightFew ? accumulate(std::integral_constant<uint32_t, kFlightFew>{})
                                                        : accumulate(std::integral_constant<uint32_t, kFlight>{});
            const uint32_t h = it.kvh * G + hg;
            if (PUSH && p.push_world) {
                const size_t rows = (size_t)p.batch * p.n_heads, rowi = (size_t)it.seq * p.n_heads + h;
                for (uint32_t r = 0; r < p.push_world; ++r) {
                    if (p.push_tagged) {
                        push::push_store(p, r, rowi * kD + d0, acc.x);
                        push::push_store(p, r, rowi * kD + d0 + 1, acc.y);
                        push::push_store(p, r, rowi * kD + d0 + 2, acc.z);
                        push::push_store(p, r, rowi * kD + d0 + 3, acc.w);
                    } else {
                        *reinterpret_cast<float4 *>(p.push_dst[r] + rowi * kD + d0) = acc;
                    }
                    if (d0 == 0) {
                        push::push_store(p, r, rows * kD + rowi, mx);
                        push::push_store(p, r, rows * kD + rows + rowi, lt);
                    }
                }
                continue;
            }
            if (p.out_acc) {
                *reinterpret_cast<float4 *>(p.out_acc + ((size_t)it.seq * p.n_heads + h) * kD + d0) = acc;
                if (d0 == 0) {
                    p.out_m[(size_t)it.seq * p.n_heads + h] = mx;
                    p.out_l[(size_t)it.seq * p.n_heads + h] = lt;
                }
                continue;
            }
            const bool ok = (fabsf(lt) <= 3.0e38f) && fabsf(lt) > 1e-6f;
            const float inv = ok ? 1.0f / lt : 0.f;  // merge rule: flash_prefill.metal:861
            float r4[4] = {acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv};
            __half *dst = p.out + (size_t)it.seq * p.out_stride_b + (size_t)h * p.out_stride_h + d0;
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) {
                if (!(fabsf(r4[i]) <= 3.0e38f)) r4[i] = 0.f;
                dst[i] = __float2half_rn(r4[i]);
            }
        }
        if (PUSH && p.push_world) push::push_signal_and_merge<(int)kD>(p, it, tid, flags);
    }
}

// Quantising append of `rows` tokens of one sequence (or one token of every sequence) into 8-bit pools: one warp
// per (token, kv head) and tensor; RoPE of k as kv_prep_fused.metal:66-82, then the row quantiser.  q rows are
// rotated into q_rot by the warps of a third group.
struct Kv8AppendParams {
    const __half *q, *k, *v;
    __half *q_rot;
    uint8_t *k_pool, *v_pool;
    float *k_scales, *v_scales;
    const __half *cos_t, *sin_t;
    const uint32_t *page_table, *kv_lens;
    uint32_t n_heads, n_kv_heads, page_size, pt_stride, n_pages, batch;
    uint32_t seq;  // 0xFFFFFFFF: one token per sequence at kv_lens[b] - 1; else `rows` tokens of sequence seq
    uint32_t position_offset, rows, rope_mode, apply_rope;
    uint32_t *status;
};

__global__ void __launch_bounds__(256) kv8_append_kernel(const Kv8AppendParams p)
{
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t wid = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t slots = p.n_heads + 2 * p.n_kv_heads;
    if (wid >= (uint64_t)p.rows * slots) return;
    const uint32_t s = (uint32_t)(wid / slots), slot = (uint32_t)(wid % slots);
    uint32_t b, pos;
    if (p.seq == 0xFFFFFFFFu) {
        b = s;
        const uint32_t len = p.kv_lens[b];
        if (len == 0) {
            if (lane == 0) atomicOr(p.status, kStatusBadPage);
            return;
        }
        pos = len - 1;
    } else {
        b = p.seq;
        pos = p.position_offset + s;
    }
    if (pos / p.page_size >= p.pt_stride) {
        if (lane == 0) atomicOr(p.status, kStatusBadPage);
        return;
    }
    const bool is_q = slot < p.n_heads, is_v = slot >= p.n_heads + p.n_kv_heads;
    const uint32_t head = is_q ? slot : (is_v ? slot - p.n_heads - p.n_kv_heads : slot - p.n_heads);
    const __half *src = is_q ? p.q + ((size_t)s * p.n_heads + head) * kD
                             : (is_v ? p.v : p.k) + ((size_t)s * p.n_kv_heads + head) * kD;
    // lane l holds dims l, l + 32, l + 64, l + 96: the NeoX mate of dim d is d + 64, the adjacent-pair mate d ^ 1
    float x[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = __half2float(src[lane + 32 * i]);
    __half y[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) y[i] = __float2half_rn(x[i]);
    if (p.apply_rope && !is_v) {
        const __half *cos_row = p.cos_t + (size_t)pos * (kD / 2), *sin_row = p.sin_t + (size_t)pos * (kD / 2);
        if (p.rope_mode == MF_ROPE_MODE_NEOX) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint32_t pr = lane + 32 * i;
                rope_pair(x[i], x[i + 2], __half2float(cos_row[pr]), __half2float(sin_row[pr]), y[i], y[i + 2]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t d = lane + 32 * i, pr = d >> 1;
                const float mate = __shfl_xor_sync(0xffffffffu, x[i], 1);
                const float cv = __half2float(cos_row[pr]), sv = __half2float(sin_row[pr]);
                __half lo, hi;
                if ((d & 1u) == 0) {
                    rope_pair(x[i], mate, cv, sv, lo, hi);
                    y[i] = lo;
                } else {
                    rope_pair(mate, x[i], cv, sv, lo, hi);
                    y[i] = hi;
                }
            }
        }
    }
    if (is_q) {
        if (!p.q_rot) return;
        __half *dst = p.seq == 0xFFFFFFFFu ? p.q_rot + ((size_t)s * p.n_heads + head) * kD
                                           : p.q_rot + ((size_t)head * p.rows + s) * kD;  // head-major packed over the rows
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[lane + 32 * i] = y[i];
        return;
    }
    const uint32_t page = p.page_table[(size_t)b * p.pt_stride + pos / p.page_size];
    if (page >= p.n_pages) {
        if (lane == 0) atomicOr(p.status, kStatusBadPage);
        return;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fabsf(__half2float(y[i])));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const float scale = amax > 0.f ? __fdiv_rn(amax, 448.f) : 1.f;
    const size_t row = ((size_t)page * p.n_kv_heads + head) * p.page_size + pos % p.page_size;
    const uint32_t in_page = pos % p.page_size;
    uint8_t *dst = is_v ? p.v_pool + (row - in_page) * kD : p.k_pool + row * kD;  // V: the page's dim-major blocks
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t d = lane + 32 * i;
        dst[is_v ? v_off8(in_page, d) : d] = (uint8_t)__nv_cvt_float_to_fp8(__fdiv_rn(__half2float(y[i]), scale), __NV_SATFINITE, __NV_E4M3);
    }
    if (lane == 0) (is_v ? p.v_scales : p.k_scales)[row] = scale;
}

// Dequantising gather: the first `len` rows of one sequence -> [Hkv, len, 128] f16 (value = f16(e4m3 * scale)).
__global__ void __launch_bounds__(256)
kv8_gather_kernel(const uint8_t *pool, const float *scales, __half *out, const uint32_t *page_table_row, uint32_t n_kv_heads,
                  uint32_t page_size, uint32_t len, uint32_t n_pages, uint32_t dim_major, uint32_t *status)
{
    const uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (uint64_t)n_kv_heads * len * kD) return;
    const uint32_t d = gid % kD, t = (gid / kD) % len, h = gid / ((uint64_t)kD * len);
    const uint32_t page = page_table_row[t / page_size];
    if (page >= n_pages) {
        atomicOr(status, kStatusBadPage);
        out[gid] = __float2half_rn(0.f);
        return;
    }
    const size_t row = ((size_t)page * n_kv_heads + h) * page_size + t % page_size;
    const uint32_t in_page = t % page_size;
    const size_t at = dim_major ? (row - in_page) * kD + v_off8(in_page, d) : row * kD + d;
    const __half_raw hr = __nv_cvt_fp8_to_halfraw(pool[at], __NV_E4M3);
    out[gid] = __float2half_rn(__half2float(__half(hr)) * scales[row]);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Byte tensor map over [rows, 128] with boxes of box_rows rows; K rows land with the 128-byte swizzle, the
// dim-major 16-key blocks of V as they are.
mf_status byte_map(MfContext *ctx, const void *base, uint64_t rows, uint32_t box_rows, bool swizzle, CUtensorMap *out)
{
    if (!ctx->encode_fn) {
        cudaDriverEntryPointQueryResult q;
        void *fn = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess || !fn)
            return fail(ctx, MF_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
        ctx->encode_fn = fn;
    }
    if (reinterpret_cast<uintptr_t>(base) & 15u) return fail(ctx, MF_ERR_INVALID_SHAPE, "8-bit pool base must be 16-byte aligned");
    cuuint64_t gdim[2] = {kD, rows};
    cuuint64_t gstride[1] = {kD};
    cuuint32_t box[2] = {kD, box_rows};
    cuuint32_t estr[2] = {1, 1};
    const CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_fn)(
        out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
        swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ctx, MF_ERR_CUDA, "cuTensorMapEncodeTiled (8-bit pool) failed (%d)", (int)r);
    return MF_OK;
}

mf_status check_kv8(MfContext *ctx, const MfPagedKv8 *c, const char *what)
{
    if (!c || !c->k_pool || !c->v_pool || !c->k_scales || !c->v_scales || !c->page_table)
        return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "%s: null pool, scales or page table", what);
    if (c->head_dim != kD) return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "%s: the 8-bit cache supports head_dim 128, got %u", what, c->head_dim);
    const uint32_t P = c->page_size;
    if (P < 16 || P > 64 || (P & (P - 1)) != 0)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "%s: page_size %u (16, 32 or 64)", what, P);
    if (c->n_kv_heads == 0 || (uint64_t)c->n_pages * c->n_kv_heads * P > 0x7FFFFFFFull)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "%s: pool geometry", what);
    if ((reinterpret_cast<uintptr_t>(c->k_scales) | reinterpret_cast<uintptr_t>(c->v_scales)) & 15u)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "%s: the scale pools must be 16-byte aligned", what);
    return MF_OK;
}

// acc / m / l: null for the whole-sequence form (rows go to a->out), else the sequence-sharded form's partials.
mf_status paged_decode_kv8_common(MfContext *ctx, const MfDecodePlan *pl, const MfPagedKv8 *c, const MfPagedDecodeArgs *a,
                                  const uint32_t *rope_positions, float *acc, float *m, float *l,
                                  const MfPeerExchange *px = nullptr, uint32_t step = 0, uint32_t merge_mask = 0)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!pl || !a) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged decode (8-bit): null argument");
    mf_status st = check_kv8(ctx, c, "paged decode (8-bit)");
    if (st != MF_OK) return st;
    if (!c->kv_lens || !a->q || (!a->out && !acc && !(px && !merge_mask)))
        return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged decode (8-bit): null tensor");
    if (px && (a->rope || a->append) && !rope_positions)
        return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged decode (8-bit): the sharded forms need rope_positions when they rotate");
    if (acc && (!m || !l || ((a->rope || a->append) && !rope_positions) || (reinterpret_cast<uintptr_t>(acc) & 15u)))
        return fail(ctx, MF_ERR_INPUT_NOT_FOUND,
                    "paged decode (8-bit): the partial form needs acc (16-byte aligned), m, l, and rope_positions when it rotates");
    if (a->append && (!a->k || !a->v)) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged decode (8-bit): k/v of the new token");
    if (a->rope && (!a->cos || !a->sin)) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged decode (8-bit): cos/sin");
    if (a->rope_mode > 1) return fail(ctx, MF_ERR_INVALID_OPERATION, "paged decode (8-bit): rope_mode %u", a->rope_mode);
    if (c->batch != pl->batch || c->n_kv_heads != pl->n_kv_heads || c->head_dim != pl->head_dim || a->n_heads != pl->n_heads ||
        c->page_size != pl->page_size)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "paged decode (8-bit): cache geometry differs from the plan");
    if (a->n_heads / c->n_kv_heads > 8)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "paged decode (8-bit): group size %u > 8", a->n_heads / c->n_kv_heads);
    if (pl->n_items == 0) return MF_OK;
    typedef void (*Kv8Kernel)(const CUtensorMap, const CUtensorMap, const Kv8Params);
    static const Kv8Kernel kernels[4] = {decode_kv8_kernel<false, false>, decode_kv8_kernel<true, false>,
                                         decode_kv8_kernel<false, true>, decode_kv8_kernel<true, true>};
    static bool configured[64] = {};
    static bool wide_clusters[64] = {};  // the cluster forms may run clusters of 16 (the non-portable size)
    if (ctx->device < 64 && !configured[ctx->device]) {
        for (int i = 0; i < 4; ++i) {
            st = check_cuda(ctx, cudaFuncSetAttribute(kernels[i], cudaFuncAttributeMaxDynamicSharedMemorySize, kDynamic),
                            "cudaFuncSetAttribute(decode, 8-bit)");
            if (st != MF_OK) return st;
        }
        wide_clusters[ctx->device] = cudaFuncSetAttribute(kernels[2], cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess &&
                                     cudaFuncSetAttribute(kernels[3], cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
        (void)cudaGetLastError();
        configured[ctx->device] = true;
    }
    Kv8Params kp{};
    DecodeParams &p = kp.d;
    p.q = static_cast<const __half *>(a->q);
    p.k_new = static_cast<const __half *>(a->k);
    p.v_new = static_cast<const __half *>(a->v);
    p.q_rot = static_cast<__half *>(a->q_rot);
    p.out = static_cast<__half *>(a->out);
    p.cos_t = static_cast<const __half *>(a->cos);
    p.sin_t = static_cast<const __half *>(a->sin);
    p.k_base = static_cast<__half *>(c->k_pool);
    p.v_base = static_cast<__half *>(c->v_pool);
    kp.k_scales = c->k_scales;
    kp.v_scales = c->v_scales;
    p.page_table = c->page_table;
    p.kv_lens = c->kv_lens;
    p.rope_positions = rope_positions;
    p.out_acc = acc;
    p.out_m = m;
    p.out_l = l;
    p.items = pl->d_items;
    p.cta_item_begin = pl->d_cta_begin;
    p.part_acc = pl->d_part_acc;
    p.part_ml = pl->d_part_ml;
    p.counters = pl->d_counters;
    p.status = ctx->d_status;
    p.n_heads = a->n_heads;
    p.n_kv_heads = c->n_kv_heads;
    p.group = a->n_heads / c->n_kv_heads;
    p.page_size = c->page_size;
    p.pt_stride = c->page_table_stride;
    p.n_pages = c->n_pages;
    p.batch = c->batch;
    p.rope = a->rope;
    p.rope_mode = a->rope_mode;
    p.append = a->append;
    p.q_stride_b = a->n_heads * kD;
    p.q_stride_h = kD;
    p.out_stride_b = a->n_heads * kD;
    p.out_stride_h = kD;
    p.knew_stride_b = c->n_kv_heads * kD;
    p.scale_log2 = a->scale * 1.4426950408889634f;
    p.early_stream = (((ctx->overlap_launches && a->append) || ctx->overlap_launches == 2) &&
                      ctx->may_stream_early(c->k_pool, c->v_pool)) ? 1u : 0u;
    if (px && (st = setup_push(ctx, px, step, merge_mask, (uint64_t)c->batch * a->n_heads, kD, p)) != MF_OK) return st;
    CUtensorMap tm_k, tm_v;
    const uint64_t rows = (uint64_t)c->n_pages * c->n_kv_heads * c->page_size;
    if ((st = byte_map(ctx, c->k_pool, rows, c->page_size, true, &tm_k)) != MF_OK) return st;
    if ((st = byte_map(ctx, c->v_pool, rows, c->page_size, false, &tm_v)) != MF_OK) return st;
    const bool programmatic = ctx->overlap_launches != 0;
    p.strict_release = (programmatic && ctx->next_launch_strict()) ? 1u : 0u;
    // A plan in the cluster form lists one range of one unit per cluster: the cluster instantiation runs it as such;
    // where the device does not take clusters of that size, every range runs as one CTA's item in the plain form
    // (correct, with fewer CTAs than the plan was made for).
    const bool clustered = pl->cluster > 1 && (pl->cluster <= 8 || (ctx->device < 64 && wide_clusters[ctx->device]));
    p.cluster_size = clustered ? pl->cluster : 1;
    p.release_late = (clustered && !p.strict_release) ? 1u : 0u;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(pl->cluster > 1 && !clustered ? pl->n_ctas / pl->cluster : pl->n_ctas);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kDynamic;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    unsigned n_attr = 0;
    if (programmatic) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (clustered) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = pl->cluster;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernels[(px ? 1 : 0) + (clustered ? 2 : 0)], tm_k, tm_v, kp);
    if (e != cudaSuccess) return fail(ctx, MF_ERR_CUDA, "launch decode_kv8_kernel: %s", cudaGetErrorString(e));
    ++ctx->launches;
    if (programmatic) ctx->note_programmatic_launch(p.strict_release != 0, a->append ? c->k_pool : nullptr, a->append ? c->v_pool : nullptr);
    return MF_OK;
}

}  // namespace
}  // namespace mf

using namespace mf;

extern "C" {

mf_status mf_paged_decode_kv8(MfContext *ctx, const MfDecodePlan *pl, const MfPagedKv8 *c, const MfPagedDecodeArgs *a)
{
    return mf::paged_decode_kv8_common(ctx, pl, c, a, nullptr, nullptr, nullptr, nullptr);
}

mf_status mf_paged_decode_kv8_push_merge(MfContext *ctx, const MfDecodePlan *pl, const MfPagedKv8 *c, const MfPagedDecodeArgs *a,
                                         const uint32_t *rope_positions, const MfPeerExchange *px, uint32_t step,
                                         uint32_t pusher_mask)
{
    if (ctx && !px) return mf::fail(ctx, MF_ERR_INPUT_NOT_FOUND, "peer exchange");
    if (ctx && !pusher_mask) return mf::fail(ctx, MF_ERR_INVALID_OPERATION, "empty pusher mask");
    if (ctx && a && !a->out) return mf::fail(ctx, MF_ERR_INPUT_NOT_FOUND, "push merge: output");
    return mf::paged_decode_kv8_common(ctx, pl, c, a, rope_positions, nullptr, nullptr, nullptr, px, step, pusher_mask);
}

mf_status mf_paged_decode_kv8_partial_push(MfContext *ctx, const MfDecodePlan *pl, const MfPagedKv8 *c, const MfPagedDecodeArgs *a,
                                           const uint32_t *rope_positions, const MfPeerExchange *px, uint32_t step)
{
    if (ctx && !px) return mf::fail(ctx, MF_ERR_INPUT_NOT_FOUND, "peer exchange");
    return mf::paged_decode_kv8_common(ctx, pl, c, a, rope_positions, nullptr, nullptr, nullptr, px, step, 0);
}

mf_status mf_paged_decode_kv8_partial(MfContext *ctx, const MfDecodePlan *pl, const MfPagedKv8 *c, const MfPagedDecodeArgs *a,
                                      const uint32_t *rope_positions, float *acc, float *m, float *l)
{
    if (ctx && (!acc || !m || !l)) return mf::fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged decode (8-bit), partial: acc / m / l");
    return mf::paged_decode_kv8_common(ctx, pl, c, a, rope_positions, acc, m, l);
}

mf_status mf_paged_kv8_append(MfContext *ctx, const MfPagedKv8 *c, const void *q, const void *k, const void *v, void *q_rot,
                              const void *cos, const void *sin, uint32_t n_heads, uint32_t rope_mode, uint32_t apply_rope,
                              uint32_t seq, uint32_t position_offset, uint32_t seq_len)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    mf_status st = check_kv8(ctx, c, "paged append (8-bit)");
    if (st != MF_OK) return st;
    if (!q || !k || !v) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged append (8-bit): q / k / v");
    if (apply_rope && (!cos || !sin)) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged append (8-bit): cos/sin");
    if (rope_mode > 1) return fail(ctx, MF_ERR_INVALID_OPERATION, "paged append (8-bit): rope_mode %u", rope_mode);
    if (n_heads == 0 || n_heads % c->n_kv_heads != 0) return fail(ctx, MF_ERR_INVALID_SHAPE, "paged append (8-bit): head counts");
    Kv8AppendParams p{};
    p.q = static_cast<const __half *>(q);
    p.k = static_cast<const __half *>(k);
    p.v = static_cast<const __half *>(v);
    p.q_rot = static_cast<__half *>(q_rot);
    p.k_pool = static_cast<uint8_t *>(c->k_pool);
    p.v_pool = static_cast<uint8_t *>(c->v_pool);
    p.k_scales = c->k_scales;
    p.v_scales = c->v_scales;
    p.cos_t = static_cast<const __half *>(cos);
    p.sin_t = static_cast<const __half *>(sin);
    p.page_table = c->page_table;
    p.kv_lens = c->kv_lens;
    p.n_heads = n_heads;
    p.n_kv_heads = c->n_kv_heads;
    p.page_size = c->page_size;
    p.pt_stride = c->page_table_stride;
    p.n_pages = c->n_pages;
    p.batch = c->batch;
    p.seq = seq;
    p.rope_mode = rope_mode;
    p.apply_rope = apply_rope;
    p.status = ctx->d_status;
    if (seq == 0xFFFFFFFFu) {
        if (!c->kv_lens) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged append (8-bit): kv_lens");
        p.rows = c->batch;
    } else {
        if (seq >= c->batch) return fail(ctx, MF_ERR_INVALID_OPERATION, "paged append (8-bit): sequence %u of %u", seq, c->batch);
        if (((uint64_t)position_offset + seq_len + c->page_size - 1) / c->page_size > c->page_table_stride)
            return fail(ctx, MF_ERR_INVALID_OPERATION, "paged append (8-bit): rows %u..%u exceed the page table", position_offset,
                        position_offset + seq_len);
        p.rows = seq_len;
        p.position_offset = position_offset;
    }
    if (p.rows == 0) return MF_OK;
    const uint64_t warps = (uint64_t)p.rows * (n_heads + 2 * c->n_kv_heads);
    kv8_append_kernel<<<(uint32_t)((warps * 32 + 255) / 256), 256, 0, ctx->stream>>>(p);
    return check_launch(ctx, "kv8_append_kernel");
}

mf_status mf_paged_kv8_gather(MfContext *ctx, const MfPagedKv8 *c, uint32_t use_v, uint32_t seq, uint32_t len, void *out)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    mf_status st = check_kv8(ctx, c, "paged gather (8-bit)");
    if (st != MF_OK) return st;
    if (!out) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged gather (8-bit): output");
    if (seq >= c->batch) return fail(ctx, MF_ERR_INVALID_OPERATION, "paged gather (8-bit): sequence %u of %u", seq, c->batch);
    if (((uint64_t)len + c->page_size - 1) / c->page_size > c->page_table_stride)
        return fail(ctx, MF_ERR_INVALID_OPERATION, "paged gather (8-bit): %u tokens exceed the page table", len);
    if (len == 0) return MF_OK;
    const uint64_t n = (uint64_t)c->n_kv_heads * len * kD;
    kv8_gather_kernel<<<(uint32_t)((n + 255) / 256), 256, 0, ctx->stream>>>(
        static_cast<const uint8_t *>(use_v ? c->v_pool : c->k_pool), use_v ? c->v_scales : c->k_scales, static_cast<__half *>(out),
        c->page_table + (size_t)seq * c->page_table_stride, c->n_kv_heads, c->page_size, len, c->n_pages, use_v ? 1u : 0u, ctx->d_status);
    return check_launch(ctx, "kv8_gather_kernel");
}

}  // extern "C"
