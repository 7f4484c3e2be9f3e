// RMSNorm -> Q/K/V projection (+bias) -> RoPE -> append for eight input rows or more, on the
// 5th-generation tensor cores (tcgen05 + TMEM).
//
// Same contract as fused_qkv_kernel (kv_append.cu; the reference's qkv_project.metal:4-272 computes
// one output row per warp with scalar FMAs): the input row is normalised and rounded to f16
// (x * inv_rms, then * gamma, both in f32), f16 x f16 products are accumulated in f32, the bias is
// added in f32, one rounding to f16, then RoPE and the stores of rope_and_store.  What differs from
// the mma.sync kernel is only the order of the f32 additions inside a dot product (the tensor core's
// own order inside a k range, the k ranges of a tile added in rank order), so a row projected with
// eight rows or more need not have the bits it has when projected alone; within this kernel the
// result of a row does not depend on how many rows travel with it.
//
// Shape of the work: a batch-sized projection is bound by the weights (31 MB for a 3B layer against
// 64 x 5120 x 3072 x 2 FLOP = 2 GFLOP).  The weight rows are the 128-row M side of the MMA, 64
// input rows its N side, the accumulator a 128 x 64 f32 tile in TMEM.  A layer has only 20-40 such
// tiles, so each tile's k range is cut over a thread-block cluster of up to eight CTAs (one CTA per
// SM pulling weights through a TMA ring of 3 to 5 stages, up to 180 KB in flight per SM); the partial tiles meet
// through distributed shared memory: CTA r of the cluster owns input rows [r * c, (r + 1) * c) of
// the tile, every CTA stores its partial sums of those rows into r's receive buffer (plain
// st.shared::cluster, coalesced over the 128 output features), one cluster barrier, and each CTA
// finishes its own rows: sum over the ranks in order, bias, f16, RoPE, stores.
//
//   warps 0-3  epilogue: warp w reads TMEM lanes 32w .. 32w + 31 (= output features)
//   warp 4     TMA producer (one thread): weight boxes of the first stages before the dependency wait
//              (weights are constants of the stream), input boxes after it
//   warp 5     TMEM allocation and the one thread that issues tcgen05.mma
//
// Weight layouts: row-major [n, k] (boxes of 64 k-elements, 128-byte swizzle) and the reference's
// blocked layout [k / 32][n][32] (boxes of 32 k-elements x 128 rows x 4 k-blocks, 64-byte swizzle).
#include <algorithm>

#include "append.cuh"
#include "internal.hpp"
#include "ptx.cuh"
#include "tcgen05.cuh"

namespace mf {
namespace {

constexpr uint32_t kTM = 128;       // output features per tile (M of the MMA)
constexpr uint32_t kTN = 64;        // input rows per tile at most (N of the MMA: 16, 32, 48 or 64)
constexpr uint32_t kStageK = 128;   // k elements per pipeline stage
constexpr uint32_t kMaxStages = 5;
constexpr uint32_t kWBytes = kTM * kStageK * 2;  // 32 KB of weights per stage
constexpr uint32_t kRingBytes = 184 * 1024;  // 5 stages at N = 16, 4 at 32 and 48, 3 at 64
constexpr uint32_t kMaxSplit = 8;   // portable cluster size
constexpr uint32_t kTcThreads = 192;
constexpr uint64_t kWaitNs = 2000000000ull;

// shared memory: the ring, the receive buffer [rank][column][128 features] f32 (columns of all ranks:
// at most kTN + kMaxSplit - 1), barriers
constexpr uint32_t kRecvCols = kTN + kMaxSplit;
constexpr uint32_t kOffRecv = kRingBytes;
constexpr uint32_t kOffBars = kOffRecv + kRecvCols * kTM * 4;
constexpr uint32_t kOffBias = kOffBars + 128;  // the tile's 128 bias values as f32
constexpr uint32_t kTcSmem = kOffBias + kTM * 4;
constexpr uint32_t kTcDynamic = kTcSmem + 1024;  // the ring is aligned to 1 KB by hand

struct QkvTcParams {
    QkvParams q;          // the fields shared with fused_qkv_kernel (x is the normalised input here)
    uint32_t split;       // CTAs per output tile along k = cluster size
    uint32_t kb_bytes;    // bytes of a row inside one TMA box = swizzle span: 64 (blocked weights) or 128
    uint32_t n_stages;    // k_dim / kStageK
    uint32_t tn;          // N of the MMA = rows of an input box: the row count of a tile rounded up to 16
    uint32_t ring;        // stages of the ring: what fits into kRingBytes at this N, at most kMaxStages
    uint32_t *status;
};

// x [m, K] -> xn [m, K]: f16(f16-widened x * inv_rms * gamma), the arithmetic and the order of the sums of
// fused_qkv_kernel (thread t squares elements 8 (t + 256 i) .., warp sums by xor shuffles, the eight warps in
// order), so that both projection kernels multiply the same normalised rows.
__global__ void __launch_bounds__(256) qkv_norm_kernel(const __half *x, const __half *gamma, __half *xn, uint32_t K, float eps,
                                                       uint32_t strict_release)
{
    __shared__ float ssq[8];
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, vecs = K / 8;
    if (!strict_release) grid_launch_dependents();
    grid_dependency_wait();
    if (strict_release) grid_launch_dependents();
    const __half *row = x + (size_t)blockIdx.x * K;
    __half *dst = xn + (size_t)blockIdx.x * K;
    float sq = 0.f;
    for (uint32_t i = tid; i < vecs; i += 256) {
        Chunk c;
        c.u = *reinterpret_cast<const uint4 *>(row + 8 * i);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float f = __half2float(c.h[e]);
            sq = fmaf(f, f, sq);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    if (lane == 0) ssq[warp] = sq;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int wv = 0; wv < 8; ++wv) t += ssq[wv];
    const float inv = 1.0f / sqrtf(t / (float)K + eps);
    for (uint32_t i = tid; i < vecs; i += 256) {
        Chunk c, g;
        c.u = *reinterpret_cast<const uint4 *>(row + 8 * i);
        g.u = *reinterpret_cast<const uint4 *>(gamma + 8 * i);
#pragma unroll
        for (int e = 0; e < 8; ++e)
            c.h[e] = __float2half_rn(__fmul_rn(__fmul_rn(__half2float(c.h[e]), inv), __half2float(g.h[e])));
        *reinterpret_cast<uint4 *>(dst + 8 * i) = c.u;
    }
}

__global__ void __launch_bounds__(kTcThreads, 1)
fused_qkv_tc_kernel(const __grid_constant__ CUtensorMap tm_wq, const __grid_constant__ CUtensorMap tm_wk,
                    const __grid_constant__ CUtensorMap tm_wv, const __grid_constant__ CUtensorMap tm_x, const QkvTcParams tp,
                    const AppendParams ap)
{
    const QkvParams &qp = tp.q;
    extern __shared__ uint8_t tc_smem_raw[];
    const uint32_t smem_base = (smem_u32(tc_smem_raw) + 1023u) & ~1023u;
    uint8_t *smem = tc_smem_raw + (smem_base - smem_u32(tc_smem_raw));
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t bars = smem_base + kOffBars;
    const uint32_t bar_full = bars, bar_empty = bars + kMaxStages * 8, bar_acc = bars + 2 * kMaxStages * 8;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + kOffBars + 96);
    const uint32_t kStages = tp.ring, tn = tp.tn;
    const uint32_t kXBytes = tn * kStageK * 2, kStageBytes = kWBytes + kXBytes;
    volatile uint32_t *abort_flag = tmem_slot + 1;

    // which tile, which k range
    const uint32_t S = tp.split, rank = S > 1 ? cluster_cta_rank() : 0u;
    const uint32_t tile = blockIdx.x / S, tiles_q = qp.n_dim / kTM, tiles_kv = qp.n_kv / kTM;
    const uint32_t mtx = tile < tiles_q ? 0u : (tile < tiles_q + tiles_kv ? 1u : 2u);
    const uint32_t row0 = (mtx == 0 ? tile : (mtx == 1 ? tile - tiles_q : tile - tiles_q - tiles_kv)) * kTM;
    const CUtensorMap *tm_w = mtx == 0 ? &tm_wq : (mtx == 1 ? &tm_wk : &tm_wv);
    const uint32_t mrow0 = blockIdx.y * kTN, mt = min(kTN, qp.m - mrow0);
    const uint32_t st0 = rank * tp.n_stages / S, st1 = (rank + 1) * tp.n_stages / S, n_local = st1 - st0;
    const uint32_t kb = tp.kb_bytes, n_sub = 256u / kb, k_steps = kb / 32u;  // boxes per stage, MMAs per box

    if (tid == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, 1);
        }
        mbar_init(bar_acc, 1);
        *abort_flag = 0;
        mbar_fence_init();
        fence_proxy_async();
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), kTN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    if (!qp.strict_release) grid_launch_dependents();

    auto wait = [&](uint32_t b, uint32_t parity, uint32_t code) {
        if (mbar_try_wait(b, parity)) return;
        if (!*abort_flag && !mbar_wait_bounded(b, parity, kWaitNs)) {
            *abort_flag = 1;
            atomicOr(tp.status, code);
        }
    };

    if (warp == 4) {
        // ------------------------------------------------------------------ TMA producer ---
        if (lane == 0) {
            tma_prefetch_desc(tm_w);
            tma_prefetch_desc(&tm_x);
            const uint64_t policy = l2_policy_evict_first();  // weights cross once
            auto load_w = [&](uint32_t i) {
                const uint32_t stage = i % kStages, dst = smem_base + stage * kStageBytes, full = bar_full + stage * 8;
                const uint32_t k0 = (st0 + i) * kStageK;
                if (kb == 64) {
                    tma_load_3d_hint(dst, tm_w, 0, (int32_t)row0, (int32_t)(k0 / 32), full, policy);  // 32 x 128 x 4 k-blocks
                } else {
                    for (uint32_t sb = 0; sb < n_sub; ++sb)
                        tma_load_2d_hint(dst + sb * (kTM * 128), tm_w, (int32_t)(k0 + 64 * sb), (int32_t)row0, full, policy);
                }
            };
            auto load_x = [&](uint32_t i) {
                const uint32_t stage = i % kStages, dst = smem_base + stage * kStageBytes + kWBytes, full = bar_full + stage * 8;
                const uint32_t k0 = (st0 + i) * kStageK;
                for (uint32_t sb = 0; sb < n_sub; ++sb)
                    tma_load_2d(dst + sb * (tn * kb), &tm_x, (int32_t)(k0 + (kb / 2) * sb), (int32_t)mrow0, full);
            };
            // the weights of the first stages travel while the kernel in front (the normalisation) still runs
            const uint32_t pre = min(n_local, kStages);
            for (uint32_t i = 0; i < pre; ++i) {
                mbar_arrive_expect_tx(bar_full + (i % kStages) * 8, kStageBytes);
                load_w(i);
            }
            grid_dependency_wait();
            for (uint32_t i = 0; i < pre; ++i) load_x(i);
            for (uint32_t i = pre; i < n_local; ++i) {
                wait(bar_empty + (i % kStages) * 8, ((i / kStages) & 1u) ^ 1u, 64u);
                if (*abort_flag) break;
                mbar_arrive_expect_tx(bar_full + (i % kStages) * 8, kStageBytes);
                load_w(i);
                load_x(i);
            }
            if (*abort_flag) {
                // nobody consumes the ring any more: let the copies in flight land before the CTA gives its memory back
                for (uint32_t s = 0; s < min(n_local, kStages); ++s) (void)mbar_wait_bounded(bar_full + s * 8, 0, kWaitNs);
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------- MMA issuer ---
        if (lane == 0) {
            const uint32_t kIdesc = instr_desc_f16(kTM, tn, 0);
            const uint32_t layout = kb == 64 ? 4u : 2u, sbo = 8u * kb;
            for (uint32_t i = 0; i < n_local; ++i) {
                const uint32_t stage = i % kStages;
                wait(bar_full + stage * 8, (i / kStages) & 1u, 128u);
                if (*abort_flag) break;
                tc_fence_after();
                const uint32_t w_addr = smem_base + stage * kStageBytes, x_addr = w_addr + kWBytes;
                for (uint32_t sb = 0; sb < n_sub; ++sb) {
                    const uint64_t a_desc = smem_desc_layout(w_addr + sb * (kTM * kb), 16, sbo, layout);
                    const uint64_t b_desc = smem_desc_layout(x_addr + sb * (tn * kb), 16, sbo, layout);
                    for (uint32_t ks = 0; ks < k_steps; ++ks)
                        tc_mma_ss(tmem, a_desc + 2 * ks, b_desc + 2 * ks, kIdesc, (i | sb | ks) != 0);  // + 32 bytes per k step
                }
                tc_commit(bar_empty + stage * 8);  // the slot is free once these products have read it
            }
            tc_commit(bar_acc);
        }
    }

    // ---------------------------------------------------------------- reduce-scatter over the cluster ---
    const uint32_t cpr = (mt + S - 1) / S;  // input rows (tile columns) owned by a rank
    const uint32_t recv = smem_base + kOffRecv;
    float *bias_s = reinterpret_cast<float *>(smem + kOffBias);
    if (warp < 4) {
        {  // the tile's bias (a constant of the stream, like the weights) while the products run
            const __half *bias = mtx == 0 ? qp.b_q : (mtx == 1 ? qp.b_k : qp.b_v);
            bias_s[tid] = bias ? __half2float(bias[row0 + tid]) : 0.f;
        }
        wait(bar_acc, 0, 256u);
        tc_fence_after();
        grid_dependency_wait();  // (has returned long ago in the producer; orders this thread's own accesses too)
        // The partial tile goes through this CTA's own ring (idle now: every product that read it has completed)
        // as [column][128 features], so that a warp hands a column to its owner with one 16-byte store per lane:
        // scalar remote stores, one per lane and column, had cost several microseconds.
        float *stage = reinterpret_cast<float *>(smem);
        if (!*abort_flag) {
            const uint32_t f = warp * 32 + lane;  // this thread's output feature = TMEM lane
#pragma unroll
            for (uint32_t half = 0; half < kTN / 32; ++half) {
                if (half * 32 < tn) {
                    uint32_t v[32];
                    tmem_ld32(tmem + ((warp * 32) << 16) + half * 32, v);
                    tc_wait_ld();
#pragma unroll
                    for (uint32_t c = 0; c < 32; ++c)
                        if (half * 32 + c < mt) stage[(half * 32 + c) * kTM + f] = __uint_as_float(v[c]);
                }
            }
        }
        named_bar_sync(1, 128);
        if (!*abort_flag) {
            for (uint32_t c = warp; c < mt; c += 4) {
                const uint32_t owner = c / cpr, cl = c - owner * cpr;
                const float4 v4 = *reinterpret_cast<const float4 *>(stage + c * kTM + 4 * lane);
                st_cluster_f4(cluster_map_shared(recv + ((rank * cpr + cl) * kTM + 4 * lane) * 4, owner), v4);
            }
        }
        tc_fence_before();
    }
    __syncwarp();
    if (S > 1) {
        cluster_arrive_release();
        cluster_wait_acquire();
    } else {
        __syncthreads();
    }
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem, kTN);
    }
    if (qp.strict_release) grid_launch_dependents();
    if (warp >= 4 || *abort_flag) return;

    // ------------------------------------------------- this rank's rows: sum, bias, f16, RoPE, stores ---
    const uint32_t my_first = rank * cpr, my_cols = my_first < mt ? min(cpr, mt - my_first) : 0u;
    const uint32_t hd = qp.head_dim, pairs_per_slot = hd / 16, pairs = kTM / 16;
    __half *plain = mtx == 0 ? qp.out_q : (mtx == 1 ? qp.out_k : qp.out_v);
    const uint32_t n_out = mtx == 0 ? qp.n_dim : qp.n_kv;
    const uint32_t slot0 = (mtx == 0 ? 0u : (mtx == 1 ? qp.q_slots : qp.q_slots + qp.kv_slots)) + row0 / hd;
    const float *rv = reinterpret_cast<const float *>(smem + kOffRecv);
    for (uint32_t item = tid; item < my_cols * pairs; item += 128) {
        const uint32_t cl = item / pairs, pr = item % pairs;
        const uint32_t sl = pr / pairs_per_slot, j = pr % pairs_per_slot;
        const uint32_t fa = sl * hd + 8 * j, fc = fa + hd / 2;  // features of the pair's two chunks inside the tile
        float4 acc[4] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f),
                         make_float4(0.f, 0.f, 0.f, 0.f)};
        for (uint32_t r = 0; r < S; ++r) {  // the ranks' k ranges, in order
            const float *src = rv + (r * cpr + cl) * kTM;
            const float4 v[4] = {*reinterpret_cast<const float4 *>(src + fa), *reinterpret_cast<const float4 *>(src + fa + 4),
                                 *reinterpret_cast<const float4 *>(src + fc), *reinterpret_cast<const float4 *>(src + fc + 4)};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                acc[q].x += v[q].x;
                acc[q].y += v[q].y;
                acc[q].z += v[q].z;
                acc[q].w += v[q].w;
            }
        }
        Chunk a, c;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 bv = *reinterpret_cast<const float4 *>(bias_s + (q < 2 ? fa : fc) + 4 * (q & 1));
            Chunk &dst = q < 2 ? a : c;
            dst.h[4 * (q & 1) + 0] = __float2half_rn(acc[q].x + bv.x);
            dst.h[4 * (q & 1) + 1] = __float2half_rn(acc[q].y + bv.y);
            dst.h[4 * (q & 1) + 2] = __float2half_rn(acc[q].z + bv.z);
            dst.h[4 * (q & 1) + 3] = __float2half_rn(acc[q].w + bv.w);
        }
        const uint32_t s = mrow0 + my_first + cl;  // input row
        if (plain) {
            __half *dst = plain + (size_t)s * n_out + row0;
            *reinterpret_cast<uint4 *>(dst + fa) = a.u;
            *reinterpret_cast<uint4 *>(dst + fc) = c.u;
        }
        if (qp.append) rope_and_store(ap, s, slot0 + sl, j, a, c);
    }
}

}  // namespace

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

namespace {

mf_status encode_f16(MfContext *ctx, CUtensorMap *out, const void *base, uint32_t rank, const cuuint64_t *dims,
                     const cuuint64_t *strides, const cuuint32_t *box, bool swizzle64, const char *what)
{
    if (!ctx->encode_fn) {
        cudaDriverEntryPointQueryResult q;
        void *fn = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess || !fn)
            return fail(ctx, MF_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
        ctx->encode_fn = fn;
    }
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_fn)(
        out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, rank, const_cast<void *>(base), dims, strides, box, estr,
        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ctx, MF_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed (%d)", what, (int)r);
    return MF_OK;
}

// Tensor map over one weight matrix [n, k]: blocked [k / 32][n][32] -> 3-D boxes of 32 x 128 rows x 4 k-blocks with
// the 64-byte swizzle (a stage's weights in one copy); row-major -> 2-D boxes of 64 x 128 rows, 128-byte swizzle.
mf_status weight_map(MfContext *ctx, CUtensorMap *out, const void *w, uint32_t n, uint32_t k, bool blocked, const char *what)
{
    if (blocked) {
        const cuuint64_t dims[3] = {32, n, k / 32};
        const cuuint64_t strides[2] = {64, (cuuint64_t)n * 64};
        const cuuint32_t box[3] = {32, kTM, kStageK / 32};
        return encode_f16(ctx, out, w, 3, dims, strides, box, true, what);
    }
    const cuuint64_t dims[2] = {k, n};
    const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    const cuuint32_t box[2] = {64, kTM};
    return encode_f16(ctx, out, w, 2, dims, strides, box, false, what);
}

}  // namespace

bool fused_qkv_tc_eligible(const MfContext *ctx, const QkvParams &qp)
{
    if (ctx->qkv_impl == 1) return false;
    if (qp.m < 8 && ctx->qkv_impl != 2) return false;  // below eight rows the mma.sync kernel's single launch is faster
    if (qp.k_dim % kStageK || qp.n_dim % kTM || qp.n_kv % kTM) return false;
    if (qp.head_dim < 16 || kTM % qp.head_dim) return false;
    return true;
}

mf_status launch_fused_qkv_tc(MfContext *ctx, QkvParams &qp, const AppendParams &ap, const char *what)
{
    const bool programmatic = ctx->overlap_launches != 0;
    const __half *x_in = qp.x;
    if (qp.gamma) {
        // normalised rows go through a buffer of the context (grown on demand: the first call of a size allocates)
        const size_t need = (size_t)qp.m * qp.k_dim * sizeof(__half);
        if (ctx->qkv_xn_bytes < need) {
            if (ctx->qkv_xn) cudaFree(ctx->qkv_xn);
            ctx->qkv_xn = nullptr;
            ctx->qkv_xn_bytes = 0;
            mf_status st = check_cuda(ctx, cudaMalloc(&ctx->qkv_xn, need), "cudaMalloc(normalised rows)");
            if (st != MF_OK) return st;
            ctx->qkv_xn_bytes = need;
        }
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(qp.m);
        cfg.blockDim = dim3(256);
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = programmatic ? 1 : 0;
        const uint32_t strict = (programmatic && ctx->next_launch_strict()) ? 1u : 0u;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, qkv_norm_kernel, qp.x, qp.gamma, static_cast<__half *>(ctx->qkv_xn), qp.k_dim,
                                                 qp.eps, strict);
        if (e != cudaSuccess) return fail(ctx, MF_ERR_CUDA, "launch qkv_norm_kernel: %s", cudaGetErrorString(e));
        ++ctx->launches;
        if (programmatic) ctx->note_programmatic_launch(strict != 0, nullptr, nullptr);
        x_in = static_cast<const __half *>(ctx->qkv_xn);
    }

    QkvTcParams tp{};
    tp.q = qp;
    tp.q.x = x_in;
    tp.kb_bytes = qp.blocked ? 64u : 128u;
    tp.n_stages = qp.k_dim / kStageK;
    tp.status = ctx->d_status;
    const uint32_t tiles = (qp.n_dim + 2 * qp.n_kv) / kTM, m_tiles = (qp.m + kTN - 1) / kTN;
    tp.tn = m_tiles > 1 ? kTN : ((qp.m + 15u) / 16u) * 16u;
    tp.ring = std::min(kMaxStages, kRingBytes / (kWBytes + tp.tn * kStageK * 2));
    static bool configured[64] = {};
    static int max_clusters[64][kMaxSplit + 1] = {};
    mf_status st;
    if (ctx->device < 64 && !configured[ctx->device]) {
        st = check_cuda(ctx, cudaFuncSetAttribute(fused_qkv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcDynamic),
                        "cudaFuncSetAttribute(fused_qkv_tc_kernel)");
        if (st != MF_OK) return st;
        // how many clusters of each size the device holds at once (a cluster needs its SMs inside one GPC)
        for (uint32_t c = 2; c <= kMaxSplit; ++c) {
            cudaLaunchConfig_t qc{};
            qc.gridDim = dim3(c);
            qc.blockDim = dim3(kTcThreads);
            qc.dynamicSmemBytes = kTcDynamic;
            cudaLaunchAttribute qa[1];
            qa[0].id = cudaLaunchAttributeClusterDimension;
            qa[0].val.clusterDim.x = c;
            qa[0].val.clusterDim.y = 1;
            qa[0].val.clusterDim.z = 1;
            qc.attrs = qa;
            qc.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, fused_qkv_tc_kernel, &qc) != cudaSuccess) n = 0;
            max_clusters[ctx->device][c] = n;
        }
        (void)cudaGetLastError();  // a refused query is an answer, not an error of this call
        configured[ctx->device] = true;
    }
    // The k range of a tile is cut over as many CTAs as keeps every cluster of the launch resident at once.
    uint32_t split = 1;
    for (uint32_t c = std::min(kMaxSplit, tp.n_stages); c >= 2; --c) {
        const int fit = ctx->device < 64 ? max_clusters[ctx->device][c] : 0;
        if ((uint32_t)fit >= tiles * m_tiles) {
            split = c;
            break;
        }
    }
    tp.split = split;

    CUtensorMap tm_wq, tm_wk, tm_wv, tm_x;
    if ((st = weight_map(ctx, &tm_wq, qp.w_q, qp.n_dim, qp.k_dim, qp.blocked != 0, what)) != MF_OK) return st;
    if ((st = weight_map(ctx, &tm_wk, qp.w_k, qp.n_kv, qp.k_dim, qp.blocked != 0, what)) != MF_OK) return st;
    if ((st = weight_map(ctx, &tm_wv, qp.w_v, qp.n_kv, qp.k_dim, qp.blocked != 0, what)) != MF_OK) return st;
    {
        const cuuint64_t dims[2] = {qp.k_dim, qp.m};
        const cuuint64_t strides[1] = {(cuuint64_t)qp.k_dim * 2};
        const cuuint32_t box[2] = {tp.kb_bytes / 2, tp.tn};
        if ((st = encode_f16(ctx, &tm_x, x_in, 2, dims, strides, box, qp.blocked != 0, what)) != MF_OK) return st;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(tiles * split, m_tiles);
    cfg.blockDim = dim3(kTcThreads);
    cfg.dynamicSmemBytes = kTcDynamic;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    uint32_t na = 0;
    if (split > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = split;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (programmatic) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
        tp.q.strict_release = ctx->next_launch_strict() ? 1u : 0u;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, fused_qkv_tc_kernel, tm_wq, tm_wk, tm_wv, tm_x, tp, ap);
    if (e != cudaSuccess) return fail(ctx, MF_ERR_CUDA, "launch fused_qkv_tc_kernel: %s", cudaGetErrorString(e));
    ++ctx->launches;
    if (programmatic)
        ctx->note_programmatic_launch(tp.q.strict_release != 0, qp.append ? ap.k_cache : nullptr, qp.append ? ap.v_cache : nullptr);
    return MF_OK;
}

}  // namespace mf
