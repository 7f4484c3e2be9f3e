// GQA flash-decode over a PAGED 8-bit (FP8 E4M3) K/V cache for sm_100a, with the append of the step's
// new token (RoPE of k, per-row quantisation) and the RoPE of q fused in.
//
// No counterpart in the reference, which only has a roadmap for a quantised cache
// (docs/FLASH.md:121-186, docs/SAGE.md:1-60).  The attention contract is the reference's
// (flash_decode.metal:146-490: q rounded to f16 after RoPE, products accumulated in f32, scores times
// `scale`, running max from -1e30, non-finite scores count as -1e30, acc / l, one rounding to f16)
// with K := the decoded bytes times the row's scale and V := the dequantised rows.
//
// Cache format (defined by this project): pools [n_pages, Hkv, P, 128] bytes for K and for V, each
// byte an OCP FP8 E4M3 value, and scale pools [n_pages, Hkv, P] f32, one scale per cached row:
//     amax = max |x_i| over the row (K after RoPE and f16 rounding, V as given),
//     scale = amax / 448 (1 for an all-zero row), byte_i = e4m3_rne_satfinite(x_i / scale).
// Half the bytes of the f16 cache cross HBM per key.
//
// Kernel shape: that of decode_kernel (decode.cu) - a TMA producer warp filling a ring of 64-key K/V
// tiles, four consumer warps of 16 keys each on mma.sync m16n8k16 with the query group on the 8-wide N
// side, equal spans of tiles per CTA from the host's plan, partials and an atomic ticket for units cut
// into several spans.  What differs:
//  * a tile row is 128 bytes, so one TMA box per page brings whole rows (128-byte swizzle), and the
//    row scales of a tile arrive by 16-byte cp.async copies that complete on the same mbarrier;
//  * ldmatrix moves the bytes as 16-bit units: for K each register holds four consecutive dims of a
//    key, which become two f16x2 operands (cvt.rn.f16x2.e4m3x2) of an MMA whose k order is permuted
//    the same way for the q fragment; for V the transposing ldmatrix delivers (key, key+1) x (dim,
//    dim+1) blocks, a byte permute separates the two dims, and the MMA's row order is permuted
//    (row r <-> dim 2r, row r+8 <-> dim 2r+1 of a 16-dim chunk), which the epilogue undoes;
//  * K's row scale multiplies the f32 score; V's row scale multiplies the softmax weight of its key,
//    relative to the largest scale among the warp's 16 keys (so the f16 weight stays in normal range),
//    and the accumulator is kept in units of that largest scale, switched inside the online-softmax
//    rescale.
#include <cuda_fp8.h>

#include "internal.hpp"
#include "ptx.cuh"

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
constexpr uint64_t kWaitLimitNs = 2000000000ull;
constexpr float kLn2 = 0.6931471805599453f;

constexpr uint32_t kTileBytes = kTileKeys * kD;  // one K or V tile: 8 KB
constexpr uint32_t kStageBytes = 2 * kTileBytes;
constexpr uint32_t kScaleStage = 2 * kTileKeys * 4;  // K scales then V scales of a tile
constexpr uint32_t kOffScales = kStages * kStageBytes;
constexpr uint32_t kCombStride = kD / 2 + 4;
constexpr uint32_t kOffComb = kOffScales + kStages * kScaleStage;
constexpr uint32_t kCombBytes = kConsumerWarps * kHP * kCombStride * 4;
constexpr uint32_t kQStride = kD + 8;
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

__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t two_bytes)
{
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(two_bytes), __NV_E4M3);
    return (uint32_t)h.x | ((uint32_t)h.y << 16);
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// The executing thread's earlier cp.async copies arrive on the mbarrier when they complete (the barrier's
// count already includes this arrival).
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar)
{
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void rope_pair(float xi, float xj, float c, float s, __half &oi, __half &oj)
{
    oi = __float2half_rn(__fsub_rn(__fmul_rn(xi, c), __fmul_rn(xj, s)));
    oj = __float2half_rn(__fadd_rn(__fmul_rn(xj, c), __fmul_rn(xi, s)));
}

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
            // per producer warp: its expect-tx arrival + one arrival per lane for the scale copies
            mbar_init(bar_full + s * 8, kProducerWarps * (1 + 32));
            mbar_init(bar_empty + s * 8, kConsumerWarps);
        }
        flags[0] = 0;
        flags[1] = 0;
        mbar_fence_init();
        fence_proxy_async();
    }
    __syncthreads();

    const uint32_t P = p.page_size;  // a power of two in 8..64
    const uint32_t boxes_per_tile = kTileKeys / P;
    if (!p.strict_release) grid_launch_dependents();

    auto row_of = [&](uint32_t seq, uint32_t kvh, uint32_t tok) -> uint32_t {
        const uint32_t page = __ldg(p.page_table + (size_t)seq * p.pt_stride + tok / P);
        return (page * p.n_kv_heads + kvh) * P + tok % P;
    };

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
        uint32_t idx = p.cta_item_begin[blockIdx.x];
        const uint32_t end = p.cta_item_begin[blockIdx.x + 1];
        uint32_t stage = 0, phase = 0, issued = 0;
        for (; idx < end; ++idx) {
            const WorkItem it = p.items[idx];
            const uint32_t L = min(p.kv_lens[it.seq], p.pt_stride * P);  // never past the page table
            for (uint32_t t = it.tile_begin; t < it.tile_end; ++t) {
                // page lookups first, then the ring slot
                const uint32_t tok_box = t * kTileKeys + lane * P;
                const bool valid = lane < boxes_per_tile && tok_box < L;
                const int32_t row_box = valid ? (int32_t)row_of(it.seq, it.kvh, tok_box) : 0;
                const uint32_t tok_sc = t * kTileKeys + 4 * lane;  // four scales per 16-byte copy, lanes 0..15
                const bool sc_valid = lane < 16 && tok_sc < L;
                const uint32_t row_sc = sc_valid ? row_of(it.seq, it.kvh, tok_sc) : 0;
                if (!flags[0] && !mbar_wait_bounded(bar_empty + stage * 8, phase ^ 1, kWaitLimitNs)) {
                    flags[0] = 1;
                    atomicOr(p.status, 1u);
                }
                const uint32_t n_valid = __popc(__ballot_sync(0xffffffffu, valid));
                const uint32_t full = bar_full + stage * 8;
                if (lane == 0) mbar_arrive_expect_tx(full, n_valid * P * kD);
                __syncwarp();
                if (valid)
                    tma_load_2d_hint(smem_base + stage * kStageBytes + (is_v ? kTileBytes : 0u) + lane * P * kD, tm, 0, row_box, full, policy);
                if (sc_valid)
                    cp_async_16(smem_base + kOffScales + stage * kScaleStage + (is_v ? kTileKeys * 4 : 0u) + lane * 16, scales + row_sc);
                cp_async_arrive_noinc(full);
                ++issued;
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
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
    float *comb = reinterpret_cast<float *>(smem + kOffComb);
    __half *q_s = reinterpret_cast<__half *>(smem + kOffQ);
    float *ml_s = reinterpret_cast<float *>(smem + kOffMl);
    __half *row_s = reinterpret_cast<__half *>(smem + kOffRow);
    float *red_s = reinterpret_cast<float *>(smem + kOffRed);
    const uint32_t G = p.group, half_d = kD / 2;
    const uint32_t g = lane >> 2, c = lane & 3;

    uint32_t idx = p.cta_item_begin[blockIdx.x];
    const uint32_t end = p.cta_item_begin[blockIdx.x + 1];
    uint32_t stage = 0, phase = 0;
    for (; idx < end; ++idx) {
        const WorkItem it = p.items[idx];
        const uint32_t L_dev = p.kv_lens[it.seq];
        const uint32_t L = min(L_dev, p.pt_stride * P);
        if (L_dev != L && tid == 0) atomicOr(p.status, kStatusBadPage);  // a length the page table has no entries for
        const uint32_t n_tiles = (L + kTileKeys - 1) / kTileKeys;
        const uint32_t pos = p.rope_positions ? p.rope_positions[it.seq] : (L ? L - 1 : 0);
        const __half *cos_row = p.cos_t + (size_t)pos * half_d, *sin_row = p.sin_t + (size_t)pos * half_d;

        // ---- q (optionally roped, rounded to f16) -> shared memory --------------------------------------
        named_bar_sync(1, kConsumerThreads);
        for (uint32_t e = tid; e < kHP * half_d; e += kConsumerThreads) {
            const uint32_t hg = e / half_d, pr = e - hg * half_d;
            const uint32_t di = p.rope_mode == MF_ROPE_MODE_NORMAL ? 2 * pr : pr;
            const uint32_t dj = p.rope_mode == MF_ROPE_MODE_NORMAL ? di + 1 : pr + half_d;
            __half oi = __float2half_rn(0.f), oj = oi;
            if (hg < G) {
                const uint32_t h = it.kvh * G + hg;
                const __half *src = p.q + (size_t)it.seq * p.q_stride_b + (size_t)h * p.q_stride_h;
                oi = src[di];
                oj = src[dj];
                if (p.rope)
                    rope_pair(__half2float(oi), __half2float(oj), __half2float(cos_row[pr]), __half2float(sin_row[pr]), oi, oj);
                if (p.q_rot && it.tile_begin == 0) {
                    __half *dst = p.q_rot + (size_t)it.seq * p.q_stride_b + (size_t)h * p.q_stride_h;
                    dst[di] = oi;
                    dst[dj] = oj;
                }
            }
            q_s[hg * kQStride + di] = oi;
            q_s[hg * kQStride + dj] = oj;
        }
        named_bar_sync(1, kConsumerThreads);
        // B fragments of Q^T for the permuted k order of the 8-bit K operand: within the 16 dims of chunk ks,
        // the MMA's k = 2c, 2c+1 are dims 4c, 4c+1 and its k = 2c+8, 2c+9 are dims 4c+2, 4c+3.
        uint32_t bq[kD / 16][2];
        {
            const __half *row = q_s + g * kQStride + 4 * c;
#pragma unroll
            for (int ks = 0; ks < (int)kD / 16; ++ks) {
                bq[ks][0] = *reinterpret_cast<const uint32_t *>(row + ks * 16);
                bq[ks][1] = *reinterpret_cast<const uint32_t *>(row + ks * 16 + 2);
            }
        }
        float m_run[2] = {kNegSentinel, kNegSentinel}, l_run[2] = {0.f, 0.f};
        float sigma = 1.f;  // the accumulators are in units of this V scale
        float o[kD / 16][4];
#pragma unroll
        for (int mt = 0; mt < (int)kD / 16; ++mt) o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f;

        for (uint32_t t = it.tile_begin; t < it.tile_end; ++t) {
            if (!flags[0] && !mbar_wait_bounded(bar_full + stage * 8, phase, kWaitLimitNs)) {
                flags[0] = 1;
                atomicOr(p.status, 2u);
            }
            uint8_t *k_tile = smem + stage * kStageBytes, *v_tile = k_tile + kTileBytes;
            const uint32_t k_addr = smem_base + stage * kStageBytes, v_addr = k_addr + kTileBytes;
            float *ksc = reinterpret_cast<float *>(smem + kOffScales + stage * kScaleStage), *vsc = ksc + kTileKeys;
            const uint32_t key0 = t * kTileKeys;
            if (t + 1 == n_tiles) {
                // The tile that holds position L - 1: quantise and splice in the token appended by this step (and
                // store it to the cache), then neutralise the rows past L (stale bytes, stale or NaN scales).
                const uint32_t r_new = (L - 1) - key0;
                bool store_ok = p.append != 0;
                uint32_t new_row = 0;
                if (p.append) {
                    const uint32_t page = p.page_table[(size_t)it.seq * p.pt_stride + (L - 1) / P];
                    store_ok = page < p.n_pages;
                    if (!store_ok && tid == 0) atomicOr(p.status, kStatusBadPage);
                    new_row = (page * p.n_kv_heads + it.kvh) * P + (L - 1) % P;
                }
                if (store_ok) {
                    const __half *ks = p.k_new + (size_t)it.seq * p.knew_stride_b + (size_t)it.kvh * kD;
                    const __half *vs = p.v_new + (size_t)it.seq * p.knew_stride_b + (size_t)it.kvh * kD;
                    if (tid < half_d) {
                        const uint32_t pr = tid;
                        const uint32_t di = p.rope_mode == MF_ROPE_MODE_NORMAL ? 2 * pr : pr;
                        const uint32_t dj = p.rope_mode == MF_ROPE_MODE_NORMAL ? di + 1 : pr + half_d;
                        __half oi = ks[di], oj = ks[dj];
                        if (p.rope)
                            rope_pair(__half2float(oi), __half2float(oj), __half2float(cos_row[pr]), __half2float(sin_row[pr]), oi, oj);
                        row_s[di] = oi;
                        row_s[dj] = oj;
                    }
                    row_s[kD + tid] = vs[tid];
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
                    reinterpret_cast<uint8_t *>(p.v_base)[(size_t)new_row * kD + tid] = qv;
                    k_tile[tile_off8(r_new, tid >> 4) + (tid & 15)] = qk;
                    v_tile[tile_off8(r_new, tid >> 4) + (tid & 15)] = qv;
                    if (tid == 0) {
                        kp.k_scales[new_row] = sk;
                        kp.v_scales[new_row] = sv;
                        ksc[r_new] = sk;
                        vsc[r_new] = sv;
                    }
                }
                const uint32_t first_dead = L - key0;  // 1..64
                for (uint32_t r = first_dead + tid; r < kTileKeys; r += kConsumerThreads) vsc[r] = 0.f;
                const uint32_t n_chunks = (kTileKeys - first_dead) * (kD / 16);
                for (uint32_t ch = tid; ch < n_chunks; ch += kConsumerThreads) {
                    const uint32_t row = first_dead + ch / (kD / 16);
                    *reinterpret_cast<uint4 *>(v_tile + tile_off8(row, ch % (kD / 16))) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async();
                named_bar_sync(2, kConsumerThreads);
            }

            const uint32_t wkey0 = key0 + warp * 16;
            if (wkey0 < L) {
                // ---- S^T (16 keys x 8 heads) = K_tile Q^T ------------------------------------------------
                float sc[4] = {0.f, 0.f, 0.f, 0.f}, sc2[4] = {0.f, 0.f, 0.f, 0.f};  // two chains: half the MMA latency exposed
                const uint32_t row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
                for (int kq = 0; kq < (int)kD / 32; ++kq) {
                    uint32_t r[4], a[4];
                    ldmatrix_x4(r, k_addr + tile_off8(row, 2 * kq + (lane >> 4)));
                    a[0] = e4m3x2_to_f16x2(r[0] & 0xFFFFu);
                    a[1] = e4m3x2_to_f16x2(r[1] & 0xFFFFu);
                    a[2] = e4m3x2_to_f16x2(r[0] >> 16);
                    a[3] = e4m3x2_to_f16x2(r[1] >> 16);
                    mma_m16n8k16(sc, a, bq[2 * kq][0], bq[2 * kq][1]);
                    a[0] = e4m3x2_to_f16x2(r[2] & 0xFFFFu);
                    a[1] = e4m3x2_to_f16x2(r[3] & 0xFFFFu);
                    a[2] = e4m3x2_to_f16x2(r[2] >> 16);
                    a[3] = e4m3x2_to_f16x2(r[3] >> 16);
                    mma_m16n8k16(sc2, a, bq[2 * kq + 1][0], bq[2 * kq + 1][1]);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) sc[i] += sc2[i];
                // ---- the rows' scales, then the online softmax over this warp's 16 keys ---------------------
                const uint32_t kr0 = wkey0 + g;
                const bool dead0 = kr0 >= L, dead1 = kr0 + 8 >= L;
                const float f0 = ksc[warp * 16 + g] * p.scale_log2, f1 = ksc[warp * 16 + g + 8] * p.scale_log2;
                float s0 = sc[0] * f0, s1 = sc[1] * f0, s2 = sc[2] * f1, s3 = sc[3] * f1;
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
                const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
                const float a0 = fast_exp2(m_run[0] - mn0), a1 = fast_exp2(m_run[1] - mn1);
                m_run[0] = mn0;
                m_run[1] = mn1;
                const float p0 = dead0 ? 0.f : fast_exp2(s0 - mn0), p1 = dead0 ? 0.f : fast_exp2(s1 - mn1);
                const float p2 = dead1 ? 0.f : fast_exp2(s2 - mn0), p3 = dead1 ? 0.f : fast_exp2(s3 - mn1);
                l_run[0] = l_run[0] * a0 + (p0 + p2);
                l_run[1] = l_run[1] * a1 + (p1 + p3);
                // V's row scales ride on the weights: weight * (scale of its key / the largest scale of these 16
                // keys) stays in f16's normal range whatever the rows' magnitudes, and the accumulator is kept in
                // units of that largest scale (sigma), switched together with the softmax rescale at no extra cost.
                const float vsa = vsc[warp * 16 + g], vsb = vsc[warp * 16 + g + 8];  // rows past L were set to 0
                float vmax = fmaxf(vsa, vsb);
#pragma unroll
                for (int off = 4; off <= 16; off <<= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, off));
                if (!(vmax > 0.f)) vmax = 1.f;
                const float inv = __frcp_rn(vmax), ra = vsa * inv, rb = vsb * inv, rs = sigma * inv;
                sigma = vmax;
                const float f0o = a0 * rs, f1o = a1 * rs;
#pragma unroll
                for (int mt = 0; mt < (int)kD / 16; ++mt) {
                    o[mt][0] *= f0o;
                    o[mt][1] *= f1o;
                    o[mt][2] *= f0o;
                    o[mt][3] *= f1o;
                }
                const uint32_t bp0 = movmatrix_trans(pack_f16x2(p0 * ra, p1 * ra)), bp1 = movmatrix_trans(pack_f16x2(p2 * rb, p3 * rb));
                // ---- O^T (dims x heads) += V_tile^T P^T: the bytes of V converted, nothing else ------------------
#pragma unroll
                for (int mp = 0; mp < (int)kD / 32; ++mp) {
                    uint32_t r[4], a[4];
                    ldmatrix_x4_trans(r, v_addr + tile_off8(row, 2 * mp + (lane >> 4)));
                    // a register: (key 2c, dims 2g, 2g+1), (key 2c+1, dims 2g, 2g+1); MMA row g <-> dim 2g, row g+8 <-> dim 2g+1
                    a[0] = e4m3x2_to_f16x2(__byte_perm(r[0], 0, 0x4420));
                    a[1] = e4m3x2_to_f16x2(__byte_perm(r[0], 0, 0x4431));
                    a[2] = e4m3x2_to_f16x2(__byte_perm(r[1], 0, 0x4420));
                    a[3] = e4m3x2_to_f16x2(__byte_perm(r[1], 0, 0x4431));
                    mma_m16n8k16(o[2 * mp], a, bp0, bp1);
                    a[0] = e4m3x2_to_f16x2(__byte_perm(r[2], 0, 0x4420));
                    a[1] = e4m3x2_to_f16x2(__byte_perm(r[2], 0, 0x4431));
                    a[2] = e4m3x2_to_f16x2(__byte_perm(r[3], 0, 0x4420));
                    a[3] = e4m3x2_to_f16x2(__byte_perm(r[3], 0, 0x4431));
                    mma_m16n8k16(o[2 * mp + 1], a, bp0, bp1);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + stage * 8);
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
#pragma unroll
        for (int hp = 0; hp < 2; ++hp) {
            {
                float *c0 = comb + (warp * kHP + 2 * c) * kCombStride, *c1 = c0 + kCombStride;
#pragma unroll
                for (int mh = 0; mh < (int)kD / 32; ++mh) {
                    const int mt = hp * (kD / 32) + mh;
                    const uint32_t d0 = mh * 16 + 2 * g;  // accumulator rows are dims 2g (first pair) and 2g + 1 (second)
                    c0[d0] = o[mt][0] * fac[0];
                    c1[d0] = o[mt][1] * fac[1];
                    c0[d0 + 1] = o[mt][2] * fac[0];
                    c1[d0 + 1] = o[mt][3] * fac[1];
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
                    const bool ok = (fabsf(l_all) <= 3.0e38f) && fabsf(l_all) > 1e-6f;
                    float r1 = ok ? acc / l_all : acc;
                    if (!(fabsf(r1) <= 3.0e38f)) r1 = 0.f;
                    const uint32_t h = it.kvh * G + hg;
                    p.out[(size_t)it.seq * p.out_stride_b + (size_t)h * p.out_stride_h + d] = __float2half_rn(r1);
                }
            }
            if (hp == 0) named_bar_sync(1, kConsumerThreads);
        }
        if (direct) continue;

        // ---- ticket: the CTA that completes the unit merges its partials (flash_prefill.metal:843-888) -------
        __threadfence();
        named_bar_sync(1, kConsumerThreads);
        if (tid == 0) {
            const uint32_t old = atomicAdd(p.counters + it.unit, 1u);
            const uint32_t last = (old + 1 == it.n_parts) ? 1u : 0u;
            if (last) p.counters[it.unit] = 0;
            flags[1] = last;
        }
        named_bar_sync(2, kConsumerThreads);
        if (!flags[1]) continue;
        __threadfence();
        for (uint32_t c4 = tid; c4 < G * (kD / 4); c4 += kConsumerThreads) {
            const uint32_t hg = c4 / (kD / 4), d0 = (c4 % (kD / 4)) * 4;
            float mx = kNegSentinel;
            for (uint32_t sp = 0; sp < it.n_parts; ++sp)
                mx = fmaxf(mx, __ldcg(p.part_ml + ((size_t)(it.first_slot + sp) * kHP + hg) * 2));
            float lt = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (uint32_t s0 = 0; s0 < it.n_parts; s0 += 8) {
                float4 v[8];
                float2 ml[8];
#pragma unroll
                for (uint32_t j = 0; j < 8; ++j) {
                    const size_t sl = it.first_slot + min(s0 + j, it.n_parts - 1);
                    v[j] = __ldcg(reinterpret_cast<const float4 *>(p.part_acc + (sl * kHP + hg) * kD + d0));
                    ml[j] = __ldcg(reinterpret_cast<const float2 *>(p.part_ml + (sl * kHP + hg) * 2));
                }
#pragma unroll
                for (uint32_t j = 0; j < 8; ++j) {
                    if (s0 + j >= it.n_parts) continue;
                    const float w = __expf(ml[j].x - mx);
                    if (ml[j].y > 0.f) lt += ml[j].y * w;
                    acc.x += v[j].x * w;
                    acc.y += v[j].y * w;
                    acc.z += v[j].z * w;
                    acc.w += v[j].w * w;
                }
            }
            const bool ok = (fabsf(lt) <= 3.0e38f) && fabsf(lt) > 1e-6f;
            const float inv = ok ? 1.0f / lt : 0.f;  // merge rule: flash_prefill.metal:861
            float r4[4] = {acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv};
            const uint32_t h = it.kvh * G + hg;
            __half *dst = p.out + (size_t)it.seq * p.out_stride_b + (size_t)h * p.out_stride_h + d0;
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) {
                if (!(fabsf(r4[i]) <= 3.0e38f)) r4[i] = 0.f;
                dst[i] = __float2half_rn(r4[i]);
            }
        }
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
    uint8_t *dst = (is_v ? p.v_pool : p.k_pool) + row * kD;
#pragma unroll
    for (int i = 0; i < 4; ++i)
        dst[lane + 32 * i] = (uint8_t)__nv_cvt_float_to_fp8(__fdiv_rn(__half2float(y[i]), scale), __NV_SATFINITE, __NV_E4M3);
    if (lane == 0) (is_v ? p.v_scales : p.k_scales)[row] = scale;
}

// Dequantising gather: the first `len` rows of one sequence -> [Hkv, len, 128] f16 (value = f16(e4m3 * scale)).
__global__ void __launch_bounds__(256)
kv8_gather_kernel(const uint8_t *pool, const float *scales, __half *out, const uint32_t *page_table_row, uint32_t n_kv_heads,
                  uint32_t page_size, uint32_t len, uint32_t n_pages, uint32_t *status)
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
    const __half_raw hr = __nv_cvt_fp8_to_halfraw(pool[row * kD + d], __NV_E4M3);
    out[gid] = __float2half_rn(__half2float(__half(hr)) * scales[row]);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Byte tensor map over [rows, 128] with boxes of box_rows rows and the 128-byte swizzle.
mf_status byte_map(MfContext *ctx, const void *base, uint64_t rows, uint32_t box_rows, CUtensorMap *out)
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
        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ctx, MF_ERR_CUDA, "cuTensorMapEncodeTiled (8-bit pool) failed (%d)", (int)r);
    return MF_OK;
}

mf_status check_kv8(MfContext *ctx, const MfPagedKv8 *c, const char *what)
{
    if (!c || !c->k_pool || !c->v_pool || !c->k_scales || !c->v_scales || !c->page_table)
        return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "%s: null pool, scales or page table", what);
    if (c->head_dim != kD) return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "%s: the 8-bit cache supports head_dim 128, got %u", what, c->head_dim);
    const uint32_t P = c->page_size;
    if (P < 8 || P > 64 || (P & (P - 1)) != 0)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "%s: page_size %u (power of two in 8..64)", what, P);
    if (c->n_kv_heads == 0 || (uint64_t)c->n_pages * c->n_kv_heads * P > 0x7FFFFFFFull)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "%s: pool geometry", what);
    return MF_OK;
}

}  // namespace
}  // namespace mf

using namespace mf;

extern "C" {

mf_status mf_paged_decode_kv8(MfContext *ctx, const MfDecodePlan *pl, const MfPagedKv8 *c, const MfPagedDecodeArgs *a)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!pl || !a) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged decode (8-bit): null argument");
    mf_status st = check_kv8(ctx, c, "paged decode (8-bit)");
    if (st != MF_OK) return st;
    if (!c->kv_lens || !a->q || !a->out) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged decode (8-bit): null tensor");
    if (a->append && (!a->k || !a->v)) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged decode (8-bit): k/v of the new token");
    if (a->rope && (!a->cos || !a->sin)) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged decode (8-bit): cos/sin");
    if (a->rope_mode > 1) return fail(ctx, MF_ERR_INVALID_OPERATION, "paged decode (8-bit): rope_mode %u", a->rope_mode);
    if (c->batch != pl->batch || c->n_kv_heads != pl->n_kv_heads || c->head_dim != pl->head_dim || a->n_heads != pl->n_heads ||
        c->page_size != pl->page_size)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "paged decode (8-bit): cache geometry differs from the plan");
    if (pl->cluster > 1)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "paged decode (8-bit): the plan is in the cluster form; create it with "
                                                         "MF_OPTION_DECODE_CLUSTERS = 1 or an explicit CTA count");
    if (a->n_heads / c->n_kv_heads > 8)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "paged decode (8-bit): group size %u > 8", a->n_heads / c->n_kv_heads);
    if (pl->n_items == 0) return MF_OK;
    static bool configured[64] = {};
    if (ctx->device < 64 && !configured[ctx->device]) {
        st = check_cuda(ctx, cudaFuncSetAttribute(decode_kv8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDynamic),
                        "cudaFuncSetAttribute(decode, 8-bit)");
        if (st != MF_OK) return st;
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
    CUtensorMap tm_k, tm_v;
    const uint64_t rows = (uint64_t)c->n_pages * c->n_kv_heads * c->page_size;
    if ((st = byte_map(ctx, c->k_pool, rows, c->page_size, &tm_k)) != MF_OK) return st;
    if ((st = byte_map(ctx, c->v_pool, rows, c->page_size, &tm_v)) != MF_OK) return st;
    const bool programmatic = ctx->overlap_launches != 0;
    p.strict_release = (programmatic && ctx->next_launch_strict()) ? 1u : 0u;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(pl->n_ctas);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kDynamic;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, decode_kv8_kernel, tm_k, tm_v, kp);
    if (e != cudaSuccess) return fail(ctx, MF_ERR_CUDA, "launch decode_kv8_kernel: %s", cudaGetErrorString(e));
    ++ctx->launches;
    if (programmatic) ctx->note_programmatic_launch(p.strict_release != 0, a->append ? c->k_pool : nullptr, a->append ? c->v_pool : nullptr);
    return MF_OK;
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
        c->page_table + (size_t)seq * c->page_table_stride, c->n_kv_heads, c->page_size, len, c->n_pages, ctx->d_status);
    return check_launch(ctx, "kv8_gather_kernel");
}

}  // extern "C"
