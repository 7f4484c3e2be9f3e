// Host side of the attention operators: argument validation, stride inference
// and routing, mirroring FlashAttentionStep / run_flash_decode of the reference
// (src/metals/sdpa/step.rs:160-503, src/metals/flashattention/step.rs:558-1086),
// plus the paged batched-decode entry points and the partial-merge kernel.
#include <algorithm>
#include <cmath>
#include <cstring>

#include "internal.hpp"

namespace mf {

mf_status launch_prefill(MfContext *ctx, const void *q, const void *k, const void *v, void *out,
                         const SdpaPrefillSplitKParams &sp, const MfPagedKv *paged = nullptr, uint32_t seq = 0);

namespace {

// acc [S, rows, D] f32, m/l [S, rows] -> out [rows, D] f16 (flash_prefill.metal:843-888).
__global__ void __launch_bounds__(128)
merge_partials_kernel(const float *__restrict__ acc, const float *__restrict__ m, const float *__restrict__ l,
                      uint32_t n_splits, uint32_t rows, uint32_t head_dim, uint64_t acc_stride, uint64_t ml_stride,
                      __half *__restrict__ out)
{
    const uint32_t row = blockIdx.x;
    float mx = -1e30f;
    for (uint32_t s = 0; s < n_splits; ++s) mx = fmaxf(mx, m[s * ml_stride + row]);
    float lt = 0.f;
    for (uint32_t s = 0; s < n_splits; ++s) {
        const float ls = l[s * ml_stride + row];
        if (ls > 0.f) lt += ls * __expf(m[s * ml_stride + row] - mx);
    }
    const float inv = ((fabsf(lt) <= 3.0e38f) && fabsf(lt) > 1e-6f) ? 1.0f / lt : 0.f;
    for (uint32_t d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float a = 0.f;
        for (uint32_t s = 0; s < n_splits; ++s)
            a += acc[s * acc_stride + (size_t)row * head_dim + d] * __expf(m[s * ml_stride + row] - mx);
        out[(size_t)row * head_dim + d] = __float2half_rn(a * inv);
    }
}

uint32_t heads_padded(uint32_t group) { return 8 * ((group + 7) / 8); }

uint64_t partial_slot_bytes(uint32_t group, uint32_t head_dim)
{
    return (uint64_t)heads_padded(group) * (head_dim + 2) * 4;
}

// Contiguous-cache decode through the shared kernel with an arithmetic plan.
// The new token's rows for the form that appends inside the decode launch (one sequence).
struct ContigAppend {
    const void *k_new, *v_new;  // [Hkv * D] each, not rotated
    void *q_rot;                // optional copy of the rotated q
    uint32_t rope_mode, apply_rope;
};

mf_status decode_contiguous(MfContext *ctx, const void *q, const void *k, const void *v, void *output,
                            const MfFlashDecodeStrides *s, const SdpaParams *sp, uint32_t n_heads, uint32_t batch,
                            uint32_t n_splits, const void *cos, const void *sin, const RopeParamsResolved *rope,
                            const ContigAppend *app = nullptr)
{
    if (!q || !k || !v || !output) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "FlashDecode: null tensor");
    if (!s || !sp) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "FlashDecode: params");
    const uint32_t D = sp->head_dim;
    if (D != 64 && D != 128)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "Flash Decode only supports head_dim=64 or 128, got %u", D);
    // The Metal kernels return without writing when the row stride differs from
    // head_dim (flash_decode.metal:165-167, 343-351); reject it instead.
    if (sp->stride_k_s != D || sp->stride_v_s != D)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "FlashDecode: K/V row stride must equal head_dim");
    if (sp->kv_len == 0 || batch == 0 || n_heads == 0) return MF_OK;  // nothing is written (flash_decode.metal:168)
    if (s->q_stride_h == 0 || s->k_stride_h == 0 || s->v_stride_h == 0)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "FlashDecode: zero head stride");
    // Head mapping of run_flash_head_layout_stage (flash_decode.metal:128-132).
    const uint32_t q_heads = std::max(1u, s->q_stride_b / s->q_stride_h);
    const uint32_t k_heads = std::max(1u, s->k_stride_b / s->k_stride_h);
    const uint32_t group = std::max(1u, q_heads / k_heads);
    if (q_heads != n_heads) return fail(ctx, MF_ERR_INVALID_SHAPE, "FlashDecode: q strides imply %u heads, n_heads=%u", q_heads, n_heads);
    if (n_heads % group != 0) return fail(ctx, MF_ERR_INVALID_SHAPE, "FlashDecode: n_heads %u not a multiple of group %u", n_heads, group);
    const uint32_t cache_heads = n_heads / group;
    if (s->k_stride_h % D || s->k_stride_b % D || s->v_stride_h % D || s->v_stride_b % D)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "FlashDecode: K/V strides must be multiples of head_dim");
    if ((uint64_t)sp->kv_len * D > s->k_stride_h || (uint64_t)sp->kv_len * D > s->v_stride_h)
        return fail(ctx, MF_ERR_INVALID_OPERATION, "FlashDecode: kv_len %u exceeds the cache capacity", sp->kv_len);

    const uint32_t T = (sp->kv_len + kTileKeys - 1) / kTileKeys;
    const uint32_t U = batch * cache_heads;
    if (U > kMaxUniformUnits) return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "FlashDecode: %u (batch x kv head) units", U);
    const uint64_t total = (uint64_t)U * T;
    if (total > 0xFFFFFFFFull) return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "FlashDecode: too many tiles");
    const uint32_t want = decode_cta_target((uint32_t)ctx->sm_count, decode_ctas_per_sm(ctx, D, group), total);
    // The cluster form only for launches of at most one CTA per SM: larger ones fill the GPU on their own, and
    // clusters, which must be placed sixteen CTAs at a time, then delay the launch behind them.
    const UniformSplit split = uniform_split(U, T, n_splits, want, want <= (uint32_t)ctx->sm_count ? decode_max_cluster(ctx, D, group) : 0u);
    const uint32_t span = split.span, n_ctas = split.n_ctas;

    const uint64_t slot_bytes = partial_slot_bytes(group, D);
    const uint64_t need = kCounterRegionBytes + (uint64_t)(U + n_ctas) * slot_bytes;
    mf_status st = ensure_scratch(ctx, need);
    if (st != MF_OK) return st;

    DecodeParams p{};
    p.q = static_cast<const __half *>(q);
    p.out = static_cast<__half *>(output);
    p.k_base = const_cast<__half *>(static_cast<const __half *>(k));
    p.v_base = const_cast<__half *>(static_cast<const __half *>(v));
    p.counters = static_cast<uint32_t *>(ctx->scratch);
    char *parts = static_cast<char *>(ctx->scratch) + kCounterRegionBytes;
    const uint32_t HP = heads_padded(group);
    p.part_acc = reinterpret_cast<float *>(parts);
    p.part_ml = reinterpret_cast<float *>(parts + (uint64_t)(U + n_ctas) * HP * D * 4);
    p.status = ctx->d_status;
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
    p.cluster_size = split.cluster;
    p.uniform_total = split.parts ? n_ctas * span : (uint32_t)total;  // the cursor turns flat / span into the CTA index
    p.q_stride_b = s->q_stride_b;
    p.q_stride_h = s->q_stride_h;
    p.out_stride_b = s->out_stride_b;
    p.out_stride_h = s->out_stride_h;
    p.scale_log2 = sp->scale * 1.4426950408889634f;
    p.rope_mode = MF_ROPE_MODE_NEOX;
    if (rope) {
        if (!cos || !sin) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "RopeFlashDecode: cos/sin");
        if (rope->dim != D) return fail(ctx, MF_ERR_INVALID_SHAPE, "RopeFlashDecode: rope dim %u != head_dim %u", rope->dim, D);
        p.rope = 1;
        p.rope_position = rope->position_offset;
        p.cos_t = static_cast<const __half *>(cos);
        p.sin_t = static_cast<const __half *>(sin);
    }
    if (app) {
        // RoPE of q and of the new key at position kv_len - 1, the new K/V rows written to the cache and
        // spliced into the last tile by the CTA that owns it: this launch is the only writer of the caches,
        // so its producers may stream ahead of the previous launch's end.
        p.append = 1;
        p.k_new = static_cast<const __half *>(app->k_new);
        p.v_new = static_cast<const __half *>(app->v_new);
        p.knew_stride_b = cache_heads * D;
        p.q_rot = static_cast<__half *>(app->q_rot);
        p.rope = app->apply_rope;
        p.rope_mode = app->rope_mode;
        p.rope_position = sp->kv_len - 1;
        p.cos_t = static_cast<const __half *>(cos);
        p.sin_t = static_cast<const __half *>(sin);
        // ... unless a launch that may still be in flight appended to this same cache (a one-layer model,
        // two calls in a row on one cache): its new row may not have landed yet
        p.early_stream = (ctx->overlap_launches && ctx->may_stream_early(k, v)) ? 1u : 0u;
    }
    // The tensor maps cover every row any (batch, head) can address.
    const uint64_t k_rows = (uint64_t)(batch - 1) * p.k_rows_b + (uint64_t)(cache_heads - 1) * p.k_rows_h + p.k_rows_h;
    const uint64_t v_rows = (uint64_t)(batch - 1) * p.v_rows_b + (uint64_t)(cache_heads - 1) * p.v_rows_h + p.v_rows_h;
    CUtensorMap tm_k, tm_v;
    // D = 128: one copy per 64-row box brings whole rows; fall back to one copy per 64-column
    // half if the driver refuses that map.
    p.whole_rows = (D == 128);
    if (p.whole_rows && (get_tensor_map(ctx, k, k_rows, D, kTileKeys, 64, &tm_k, 1) != MF_OK ||
                         get_tensor_map(ctx, v, v_rows, D, kTileKeys, 64, &tm_v, 1) != MF_OK))
        p.whole_rows = 0;
    if (!p.whole_rows) {
        if ((st = get_tensor_map(ctx, k, k_rows, D, kTileKeys, 64, &tm_k)) != MF_OK) return st;
        if ((st = get_tensor_map(ctx, v, v_rows, D, kTileKeys, 64, &tm_v)) != MF_OK) return st;
    }
    return launch_decode(ctx, tm_k, tm_v, p, D, n_ctas, app ? k : nullptr, app ? v : nullptr);
}

struct QLayout {
    uint32_t stride_b, stride_h, stride_m;
};

// The reference picks split-K from the sequence lengths alone (tuned on Apple GPUs, where one
// threadgroup per 32 rows and head is all the parallelism there is).  Here the split is only
// taken when the unsplit grid would leave SMs idle.
uint32_t effective_prefill_split_k(const MfContext *ctx, uint32_t kv_seq_len, uint32_t q_seq_len, uint32_t n_heads)
{
    const uint64_t ctas = (uint64_t)((q_seq_len + 63) / 64) * n_heads;
    if (ctas >= (uint64_t)ctx->sm_count) return 1;
    return mf_prefill_split_k(kv_seq_len, q_seq_len);
}

}  // namespace
}  // namespace mf

using namespace mf;

extern "C" {

mf_status mf_merge_partials(MfContext *ctx, const float *acc, const float *m, const float *l, uint32_t n_splits,
                            uint32_t rows, uint32_t head_dim, void *out)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!acc || !m || !l || !out) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "merge: null input");
    if (n_splits == 0 || rows == 0 || head_dim == 0) return MF_OK;
    merge_partials_kernel<<<rows, 128, 0, ctx->stream>>>(acc, m, l, n_splits, rows, head_dim, (uint64_t)rows * head_dim,
                                                         (uint64_t)rows, static_cast<__half *>(out));
    return check_launch(ctx, "merge_partials_kernel");
}

mf_status mf_merge_partials_strided(MfContext *ctx, const float *acc, const float *m, const float *l, uint32_t n_splits,
                                    uint32_t rows, uint32_t head_dim, uint64_t split_stride, void *out)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!acc || !m || !l || !out) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "merge: null input");
    if (n_splits == 0 || rows == 0 || head_dim == 0) return MF_OK;
    merge_partials_kernel<<<rows, 128, 0, ctx->stream>>>(acc, m, l, n_splits, rows, head_dim, split_stride, split_stride,
                                                         static_cast<__half *>(out));
    return check_launch(ctx, "merge_partials_kernel");
}

mf_status mf_flash_decode(MfContext *ctx, const void *q, const void *k, const void *v, void *output,
                          const MfFlashDecodeStrides *strides, const SdpaParams *params, uint32_t n_heads,
                          uint32_t batch, uint32_t n_splits)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    return decode_contiguous(ctx, q, k, v, output, strides, params, n_heads, batch, n_splits, nullptr, nullptr, nullptr);
}

mf_status mf_rope_flash_decode(MfContext *ctx, const void *q, const void *k, const void *v, const void *cos,
                               const void *sin, void *output, const RopeParamsResolved *rope, const SdpaParams *params,
                               const MfFlashDecodeStrides *strides, uint32_t n_heads, uint32_t batch)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!rope) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "RopeFlashDecode: rope params");
    return decode_contiguous(ctx, q, k, v, output, strides, params, n_heads, batch, 0, cos, sin, rope);
}

mf_status mf_flash_prefill(MfContext *ctx, const void *q, const void *k, const void *v, void *output,
                           const SdpaPrefillSplitKParams *params)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!q || !k || !v || !output) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "FlashPrefill: null tensor");
    if (!params) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "FlashPrefill: params");
    return launch_prefill(ctx, q, k, v, output, *params);
}

// run_flash_decode (src/metals/flashattention/step.rs:558-1086).
// general_offset < 0: the reference's flash routes (decode for one row, causal prefill with
// query_offset = kv_len - q_len).  general_offset >= 0: the tiled kernels with that visibility rule
// (key k visible to row r iff k <= r + general_offset), also for one row.
static mf_status run_flash_decode_impl(MfContext *ctx, const MfTensor *q, const MfTensor *k, const MfTensor *v,
                                       const MfTensor *output, uint32_t n_heads, uint32_t head_dim, uint32_t kv_seq_len,
                                       uint32_t q_seq_len, uint32_t kv_head_major, int64_t general_offset)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    mf_status st;
    if ((st = need_tensor(ctx, q, "q")) != MF_OK) return st;
    if ((st = need_tensor(ctx, k, "k")) != MF_OK) return st;
    if ((st = need_tensor(ctx, v, "v")) != MF_OK) return st;
    if ((st = need_tensor(ctx, output, "output")) != MF_OK) return st;
    if (!kv_head_major)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "FlashAttention only supports kv_head_major=true for now");
    const uint32_t D = head_dim;
    auto last_contig = [&](const MfTensor *t, const char *name) -> mf_status {
        if (t->strides[t->rank - 1] != 1)
            return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "requires contiguous last dim for %s", name);
        return MF_OK;
    };
    // n_kv_heads from the cache tensor (step.rs:430-446).
    const uint32_t n_kv_heads = std::max<uint32_t>(1, (uint32_t)(k->rank == 3 ? k->dims[0] : k->dims[1]));

    if (q_seq_len > 1 || general_offset >= 0) {
        if (D != 64 && D != 128)
            return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "Prefill only supports head_dim=64 or 128, got %u", D);
        if ((st = last_contig(q, "q")) != MF_OK) return st;
        if ((st = last_contig(k, "k")) != MF_OK) return st;
        if ((st = last_contig(v, "v")) != MF_OK) return st;
        if ((st = last_contig(output, "output")) != MF_OK) return st;
        const uint64_t dm = (uint64_t)n_heads * D, M = q_seq_len;
        // Q layout inference (step.rs:658-720).  A [1, M_cap, d_model] tensor is read as
        // head-major packed over the true M, the order KvPrepFused writes.
        QLayout ql{};
        const uint64_t *qd = q->dims, *qs = q->strides;
        if (q->rank == 3 && qd[0] == 1 && qd[2] == dm) {
            ql = {n_heads * q_seq_len * D, q_seq_len * D, D};
        } else if (q->rank == 3 && qd[0] == n_heads && qd[1] >= M && qd[2] == D) {
            ql = {0, (uint32_t)qs[0], (uint32_t)qs[1]};
        } else if (q->rank == 4 && qd[1] == n_heads && qd[2] >= M && qd[3] == D) {
            ql = {(uint32_t)qs[0], (uint32_t)qs[1], (uint32_t)qs[2]};
        } else if (q->rank == 2 && qd[0] >= M && qd[1] == dm) {
            ql = {0, D, (uint32_t)qs[0]};
        } else if (q->rank == 3 && qd[1] >= M && qd[2] == dm) {
            ql = {(uint32_t)qs[0], D, (uint32_t)qs[1]};
        } else if (q->rank == 3 && qd[0] >= M && qd[1] == n_heads && qd[2] == D) {
            ql = {0, (uint32_t)qs[1], (uint32_t)qs[0]};
        } else if (q->rank == 4 && qd[1] >= M && qd[2] == n_heads && qd[3] == D) {
            ql = {(uint32_t)qs[0], (uint32_t)qs[2], (uint32_t)qs[1]};
        } else {
            return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "Prefill Q layout unsupported");
        }
        // Output layout (step.rs:722-756).
        QLayout ol{};
        const uint64_t *od = output->dims, *os = output->strides;
        if (output->rank == 2 && od[0] >= M && od[1] == dm) {
            ol = {0, D, (uint32_t)os[0]};
        } else if (output->rank == 3 && od[1] >= M && od[2] == dm) {
            ol = {(uint32_t)os[0], D, (uint32_t)os[1]};
        } else if (output->rank == 3 && od[0] >= M && od[1] == n_heads && od[2] == D) {
            ol = {0, (uint32_t)os[1], (uint32_t)os[0]};
        } else if (output->rank == 4 && od[1] >= M && od[2] == n_heads && od[3] == D) {
            ol = {(uint32_t)os[0], (uint32_t)os[2], (uint32_t)os[1]};
        } else if (output->rank == 3 && od[0] == n_heads && od[1] >= M && od[2] == D) {
            ol = {0, (uint32_t)os[0], (uint32_t)os[1]};
        } else if (output->rank == 4 && od[1] == n_heads && od[2] >= M && od[3] == D) {
            ol = {(uint32_t)os[0], (uint32_t)os[1], (uint32_t)os[2]};
        } else {
            return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "Prefill output layout unsupported");
        }
        SdpaPrefillSplitKParams pp{};
        SdpaPrefillParams &b = pp.base;
        b.kv_len = kv_seq_len;
        b.head_dim = D;
        b.scale = 1.0f / sqrtf((float)D);
        if (k->rank == 4) {
            b.k_stride_b = (uint32_t)k->strides[0];
            b.k_stride_h = (uint32_t)k->strides[1];
            b.stride_k_s = (uint32_t)k->strides[2];
        } else {
            b.k_stride_b = 0;
            b.k_stride_h = (uint32_t)k->strides[0];
            b.stride_k_s = (uint32_t)k->strides[1];
        }
        if (v->rank == 4) {
            b.v_stride_b = (uint32_t)v->strides[0];
            b.v_stride_h = (uint32_t)v->strides[1];
            b.stride_v_s = (uint32_t)v->strides[2];
        } else {
            b.v_stride_b = 0;
            b.v_stride_h = (uint32_t)v->strides[0];
            b.stride_v_s = (uint32_t)v->strides[1];
        }
        b.query_offset = general_offset >= 0 ? (uint32_t)general_offset : (kv_seq_len > q_seq_len ? kv_seq_len - q_seq_len : 0);
        b.q_stride_b = ql.stride_b;
        b.q_stride_h = ql.stride_h;
        b.q_stride_m = ql.stride_m;
        b.out_stride_b = ol.stride_b;
        b.out_stride_h = ol.stride_h;
        b.out_stride_m = ol.stride_m;
        b.group_size = std::max(1u, n_heads / n_kv_heads);
        b.q_len = q_seq_len;
        pp.n_heads = n_heads;
        pp.split_k = effective_prefill_split_k(ctx, kv_seq_len, q_seq_len, n_heads);
        return launch_prefill(ctx, tensor_ptr(q), tensor_ptr(k), tensor_ptr(v), tensor_ptr(output), pp);
    }

    // Decode: strides from the resolved sizes, not from the q tensor's metadata
    // (step.rs:995-1040).
    if (D != 64 && D != 128)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "Flash Decode only supports head_dim=64 or 128, got %u", D);
    const uint32_t capacity = k->rank >= 2 ? (uint32_t)k->dims[1] : kv_seq_len;
    MfFlashDecodeStrides s{};
    s.q_stride_b = n_heads * D;
    s.q_stride_h = D;
    s.k_stride_b = n_kv_heads * capacity * D;
    s.k_stride_h = capacity * D;
    s.v_stride_b = s.k_stride_b;
    s.v_stride_h = s.k_stride_h;
    s.out_stride_b = n_heads * D;
    s.out_stride_h = D;
    SdpaParams sp{kv_seq_len, D, 1.0f / sqrtf((float)D), D, D};
    return decode_contiguous(ctx, tensor_ptr(q), tensor_ptr(k), tensor_ptr(v), tensor_ptr(output), &s, &sp, n_heads, 1,
                             0, nullptr, nullptr, nullptr);
}

mf_status mf_run_flash_decode(MfContext *ctx, const MfTensor *q, const MfTensor *k, const MfTensor *v,
                              const MfTensor *output, uint32_t n_heads, uint32_t head_dim, uint32_t kv_seq_len,
                              uint32_t q_seq_len, uint32_t kv_head_major)
{
    return run_flash_decode_impl(ctx, q, k, v, output, n_heads, head_dim, kv_seq_len, q_seq_len, kv_head_major, -1);
}

// KvPrepFused (src/metals/kv_prep/step.rs:93-132) and the decode route of FlashAttention
// (src/metals/sdpa/step.rs:160-503) for ONE new token on a compact contiguous cache, in one launch.
mf_status mf_kv_prep_flash_decode(MfContext *ctx, const MfTensor *q, const MfTensor *k, const MfTensor *v,
                                  const MfTensor *q_rot, const MfTensor *k_cache, const MfTensor *v_cache,
                                  const MfTensor *cos, const MfTensor *sin, const MfTensor *output,
                                  const KvPrepFusedParamsResolved *pr)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!pr) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "KvPrepFused+FlashDecode: params");
    mf_status st;
    const MfTensor *ts[8] = {q, k, v, k_cache, v_cache, cos, sin, output};
    const char *names[8] = {"q", "k", "v", "k_cache", "v_cache", "cos", "sin", "output"};
    for (int i = 0; i < 8; ++i)
        if ((st = need_tensor(ctx, ts[i], names[i])) != MF_OK) return st;
    const uint32_t D = pr->head_dim;
    if (pr->seq_len != 1)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "KvPrepFused+FlashDecode: one new token per call, got %u", pr->seq_len);
    if (D != 64 && D != 128)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "Flash Decode only supports head_dim=64 or 128, got %u", D);
    if (pr->n_kv_heads == 0 || pr->n_heads % pr->n_kv_heads != 0 || pr->group_size != pr->n_heads / pr->n_kv_heads ||
        pr->d_model != pr->n_heads * D || pr->kv_dim != pr->n_kv_heads * D)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "KvPrepFused+FlashDecode: head geometry");
    if (pr->position_offset >= pr->max_seq_len)
        return fail(ctx, MF_ERR_INVALID_OPERATION, "KvPrepFused+FlashDecode: position %u outside the cache of %u rows",
                    pr->position_offset, pr->max_seq_len);
    if (pr->rope_mode > 1) return fail(ctx, MF_ERR_INVALID_OPERATION, "KvPrepFused+FlashDecode: rope_mode %u", pr->rope_mode);
    if (k_cache->rank != 3 || v_cache->rank != 3 || k_cache->dims[1] != pr->max_seq_len || k_cache->dims[2] != D ||
        v_cache->dims[0] != k_cache->dims[0] || v_cache->dims[1] != k_cache->dims[1] || v_cache->dims[2] != D)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "KvPrepFused+FlashDecode: caches must be rank-3 [heads, max_seq_len, head_dim]");
    if (k_cache->dims[0] != pr->n_kv_heads)  // an expanded cache takes G writes per row: the two-call form does that
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "KvPrepFused+FlashDecode: compact cache only (%llu heads, %u kv heads)",
                    (unsigned long long)k_cache->dims[0], pr->n_kv_heads);
    const void *ptrs[9] = {tensor_ptr(q), tensor_ptr(k), tensor_ptr(v), tensor_ptr(k_cache), tensor_ptr(v_cache),
                           tensor_ptr(cos), tensor_ptr(sin), tensor_ptr(output), q_rot ? tensor_ptr(q_rot) : nullptr};
    for (const void *ptr : ptrs)
        if (reinterpret_cast<uintptr_t>(ptr) & 15u)
            return fail(ctx, MF_ERR_INVALID_SHAPE, "KvPrepFused+FlashDecode: 16-byte alignment");
    const uint32_t cap = pr->max_seq_len, kv_len = pr->position_offset + 1;
    MfFlashDecodeStrides s{};
    s.q_stride_b = pr->n_heads * D;
    s.q_stride_h = D;
    s.k_stride_b = pr->n_kv_heads * cap * D;
    s.k_stride_h = cap * D;
    s.v_stride_b = s.k_stride_b;
    s.v_stride_h = s.k_stride_h;
    s.out_stride_b = pr->n_heads * D;
    s.out_stride_h = D;
    SdpaParams sp{kv_len, D, 1.0f / sqrtf((float)D), D, D};
    ContigAppend app{};
    app.k_new = ptrs[1];
    app.v_new = ptrs[2];
    app.q_rot = const_cast<void *>(ptrs[8]);
    app.rope_mode = pr->rope_mode;
    // SmolLM3-style skip: no RoPE on every N-th layer (kv_prep_fused.metal:56-57)
    app.apply_rope = pr->no_rope_layer_step == 0 || ((pr->layer_idx + 1u) % pr->no_rope_layer_step) != 0u;
    return decode_contiguous(ctx, ptrs[0], ptrs[3], ptrs[4], const_cast<void *>(ptrs[7]), &s, &sp, pr->n_heads, 1, 0,
                             ptrs[5], ptrs[6], nullptr, &app);
}

// SdpaReferenceStep (src/metals/sdpa/step.rs:89-158, 558-779): attention for the cases the flash routes
// refuse.  The reference materialises S and P in f16 scratch; here the same result comes from the tiled
// kernels with the general visibility rule, without scratch and with f32 softmax.
mf_status mf_sdpa_reference(MfContext *ctx, const MfTensor *q, const MfTensor *k, const MfTensor *v,
                            const MfTensor *output, const MfFlashAttentionArgs *a)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!a) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "SdpaReference: args");
    if (a->kv_seq_len == 0) return MF_OK;
    // mask rule of softmax_sdpa_batched.metal:25-37: causal hides keys i > row + query_offset
    const int64_t offset = a->causal ? (int64_t)a->query_offset : (int64_t)a->kv_seq_len;
    return run_flash_decode_impl(ctx, q, k, v, output, a->n_heads, a->head_dim, a->kv_seq_len, std::max(1u, a->m), 1, offset);
}

// FlashAttentionStep dispatcher (src/metals/sdpa/step.rs:160-503).
mf_status mf_flash_attention(MfContext *ctx, const MfTensor *q, const MfTensor *k, const MfTensor *v,
                             const MfTensor *output, const MfFlashAttentionArgs *a, uint32_t *route_out)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!a) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "FlashAttention: args");
    if (route_out) *route_out = 0;
    mf_status st;
    if ((st = need_tensor(ctx, q, "q")) != MF_OK) return st;
    if ((st = need_tensor(ctx, k, "k")) != MF_OK) return st;
    if ((st = need_tensor(ctx, v, "v")) != MF_OK) return st;
    if ((st = need_tensor(ctx, output, "output")) != MF_OK) return st;
    const uint32_t m = std::max(1u, a->m);
    if (!a->kv_head_major)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "FlashAttention only supports kv_head_major=true for now");
    if (m == 1) {
        // Online path only when nothing has to be masked (sdpa/step.rs:271).
        if (a->causal && a->query_offset + 1 != a->kv_seq_len) {
            // "FlashAttention m=1 but causal offset mismatch; falling back" (sdpa/step.rs:271-303)
            if (route_out) *route_out = MF_ROUTE_REFERENCE;
            return mf_sdpa_reference(ctx, q, k, v, output, a);
        }
        // Token-major row check (sdpa/step.rs:305-349).
        const uint64_t dm = (uint64_t)a->n_heads * a->head_dim;
        auto row_ok = [&](const MfTensor *t) {
            if (t->rank == 1) return t->dims[0] == dm;
            const uint32_t r = t->rank;
            if (r == 2 && t->dims[0] == 1 && t->dims[1] == dm) return true;
            return t->dims[r - 1] == dm && t->strides[r - 1] == 1 && t->strides[r - 2] == dm;
        };
        if (!row_ok(q) || !row_ok(output))
            return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "FlashAttention requested but tensor layout unsupported");
        if (route_out) *route_out = MF_ROUTE_DECODE;
        return mf_run_flash_decode(ctx, q, k, v, output, a->n_heads, a->head_dim, a->kv_seq_len, 1, a->kv_head_major);
    }
    if (!a->causal || a->query_offset + m != a->kv_seq_len) {
        // non-causal, or the causal invariant does not hold: the reference falls back (sdpa/step.rs:442-470)
        if (route_out) *route_out = MF_ROUTE_REFERENCE;
        return mf_sdpa_reference(ctx, q, k, v, output, a);
    }
    if (route_out)
        *route_out = effective_prefill_split_k(ctx, a->kv_seq_len, m, a->n_heads) > 1 ? MF_ROUTE_PREFILL_SPLITK
                                                                                      : MF_ROUTE_PREFILL;
    return mf_run_flash_decode(ctx, q, k, v, output, a->n_heads, a->head_dim, a->kv_seq_len, m, a->kv_head_major);
}

// ------------------------------------------------------------------ paged ---

static mf_status plan_upload(MfContext *ctx, MfDecodePlan *pl)
{
    pl->n_items = (uint32_t)pl->h_items.size();
    pl->n_ctas = ((uint32_t)pl->h_cta_begin.size() - 1) * (pl->cluster > 1 ? pl->cluster : 1);  // cluster form: one entry per cluster
    if (pl->n_items > pl->item_capacity)
        return fail(ctx, MF_ERR_INVALID_OPERATION, "decode plan: %u items exceed capacity %u", pl->n_items, pl->item_capacity);
    if (pl->n_items == 0) return MF_OK;
    const uint32_t s = pl->next_stage;
    pl->next_stage ^= 1;
    // The copy that last read this staging set must have finished.
    mf_status st = check_cuda(ctx, cudaEventSynchronize(pl->staged[s]), "cudaEventSynchronize(plan staging)");
    if (st != MF_OK) return st;
    std::memcpy(pl->pinned_items[s], pl->h_items.data(), sizeof(WorkItem) * pl->n_items);
    const size_t begin_bytes = 4 * pl->h_cta_begin.size();  // cluster form: one entry per cluster, not per CTA
    std::memcpy(pl->pinned_cta_begin[s], pl->h_cta_begin.data(), begin_bytes);
    st = check_cuda(ctx, cudaMemcpyAsync(pl->d_items, pl->pinned_items[s], sizeof(WorkItem) * pl->n_items,
                                         cudaMemcpyHostToDevice, ctx->stream), "plan upload");
    if (st != MF_OK) return st;
    st = check_cuda(ctx, cudaMemcpyAsync(pl->d_cta_begin, pl->pinned_cta_begin[s], begin_bytes,
                                         cudaMemcpyHostToDevice, ctx->stream), "plan upload");
    if (st != MF_OK) return st;
    return check_cuda(ctx, cudaEventRecord(pl->staged[s], ctx->stream), "cudaEventRecord(plan staging)");
}

mf_status mf_decode_plan_create(MfContext *ctx, const uint32_t *kv_lens_host, uint32_t batch, uint32_t n_heads,
                                uint32_t n_kv_heads, uint32_t head_dim, uint32_t page_size, uint32_t max_ctas,
                                MfDecodePlan **out)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!kv_lens_host || !out) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "decode plan: null input");
    *out = nullptr;
    if (batch == 0 || n_kv_heads == 0 || n_heads % n_kv_heads != 0)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "decode plan: batch %u, n_heads %u, n_kv_heads %u", batch, n_heads, n_kv_heads);
    if (head_dim != 64 && head_dim != 128)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "Flash Decode only supports head_dim=64 or 128, got %u", head_dim);
    if (n_heads / n_kv_heads > 16)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "decode plan: group size %u > 16", n_heads / n_kv_heads);
    const bool auto_ctas = (max_ctas == 0);
    if (auto_ctas) max_ctas = (uint32_t)ctx->sm_count * decode_ctas_per_sm(ctx, head_dim, n_heads / n_kv_heads);
    MfDecodePlan *pl = new MfDecodePlan();
    pl->batch = batch;
    pl->n_heads = n_heads;
    pl->n_kv_heads = n_kv_heads;
    pl->head_dim = head_dim;
    pl->page_size = page_size;
    pl->max_ctas = max_ctas;
    pl->auto_ctas = auto_ctas;
    pl->ctas_per_sm = decode_ctas_per_sm(ctx, head_dim, n_heads / n_kv_heads);
    pl->sm_count = (uint32_t)ctx->sm_count;
    pl->max_cluster = decode_max_cluster(ctx, head_dim, n_heads / n_kv_heads);
    pl->n_units = batch * n_kv_heads;
    pl->item_capacity = pl->n_units + max_ctas;
    pl->heads_padded = heads_padded(n_heads / n_kv_heads);
    cudaError_t e = cudaSuccess;
    auto ok = [&](cudaError_t r) {
        if (e == cudaSuccess) e = r;
    };
    for (int i = 0; i < 2; ++i) {
        ok(cudaMallocHost(reinterpret_cast<void **>(&pl->pinned_items[i]), sizeof(WorkItem) * pl->item_capacity));
        ok(cudaMallocHost(reinterpret_cast<void **>(&pl->pinned_cta_begin[i]), 4 * (max_ctas + 1)));
        ok(cudaEventCreateWithFlags(&pl->staged[i], cudaEventDisableTiming));
    }
    ok(cudaMalloc(reinterpret_cast<void **>(&pl->d_items), sizeof(WorkItem) * pl->item_capacity));
    ok(cudaMalloc(reinterpret_cast<void **>(&pl->d_cta_begin), 4 * (max_ctas + 1)));
    ok(cudaMalloc(reinterpret_cast<void **>(&pl->d_part_acc), (size_t)pl->item_capacity * pl->heads_padded * head_dim * 4));
    ok(cudaMalloc(reinterpret_cast<void **>(&pl->d_part_ml), (size_t)pl->item_capacity * pl->heads_padded * 2 * 4));
    ok(cudaMalloc(reinterpret_cast<void **>(&pl->d_counters), 4 * (size_t)pl->n_units));
    if (e == cudaSuccess) ok(cudaMemsetAsync(pl->d_counters, 0, 4 * (size_t)pl->n_units, ctx->stream));
    if (e != cudaSuccess) {
        mf_decode_plan_destroy(ctx, pl);
        return check_cuda(ctx, e, "decode plan allocation");
    }
    mf_status st = mf_decode_plan_update(ctx, pl, kv_lens_host);
    if (st != MF_OK) {
        mf_decode_plan_destroy(ctx, pl);
        return st;
    }
    *out = pl;
    return MF_OK;
}

mf_status mf_decode_plan_update(MfContext *ctx, MfDecodePlan *pl, const uint32_t *kv_lens_host)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!pl || !kv_lens_host) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "decode plan: null input");
    uint32_t ctas = pl->max_ctas;
    if (pl->auto_ctas) {
        uint64_t total = 0;
        for (uint32_t b = 0; b < pl->batch; ++b) total += (uint64_t)((kv_lens_host[b] + kTileKeys - 1) / kTileKeys) * pl->n_kv_heads;
        ctas = decode_cta_target(pl->sm_count, pl->ctas_per_sm, total);
    }
    // the cluster form only for plans whose CTA count the library chooses (an explicit count is a request for
    // exactly that many spans)
    // ... and for launches of at most one CTA per SM: larger ones fill the GPU on their own, and clusters, which
    // must be placed sixteen CTAs at a time, then delay the launch behind them
    pl->cluster = (pl->auto_ctas && ctas <= pl->sm_count) ? pl->max_cluster : 0;
    build_decode_plan(kv_lens_host, pl->batch, pl->n_kv_heads, ctas, pl->h_items, pl->h_cta_begin, &pl->n_units,
                      &pl->total_tiles, &pl->cluster, ctx->plan_item_cost);
    return plan_upload(ctx, pl);
}

void mf_decode_plan_destroy(MfContext *ctx, MfDecodePlan *pl)
{
    if (!pl) return;
    if (ctx && ctx->stream) cudaStreamSynchronize(ctx->stream);
    for (int i = 0; i < 2; ++i) {
        if (pl->pinned_items[i]) cudaFreeHost(pl->pinned_items[i]);
        if (pl->pinned_cta_begin[i]) cudaFreeHost(pl->pinned_cta_begin[i]);
        if (pl->staged[i]) cudaEventDestroy(pl->staged[i]);
    }
    if (pl->d_items) cudaFree(pl->d_items);
    if (pl->d_cta_begin) cudaFree(pl->d_cta_begin);
    if (pl->d_part_acc) cudaFree(pl->d_part_acc);
    if (pl->d_part_ml) cudaFree(pl->d_part_ml);
    if (pl->d_counters) cudaFree(pl->d_counters);
    delete pl;
}

uint32_t mf_decode_plan_build_host(const uint32_t *kv_lens_host, uint32_t batch, uint32_t n_kv_heads, uint32_t max_ctas,
                                   uint32_t *items_out, uint32_t item_capacity, uint32_t *cta_begin_out,
                                   uint32_t *n_ctas_out)
{
    if (!kv_lens_host || max_ctas == 0 || n_kv_heads == 0) return 0;
    std::vector<WorkItem> items;
    std::vector<uint32_t> cta_begin;
    uint32_t n_units = 0;
    uint64_t total = 0;
    build_decode_plan(kv_lens_host, batch, n_kv_heads, max_ctas, items, cta_begin, &n_units, &total);
    if (n_ctas_out) *n_ctas_out = (uint32_t)cta_begin.size() - 1;
    if (items.size() <= item_capacity && items_out && cta_begin_out) {
        static_assert(sizeof(WorkItem) == 32, "WorkItem is 8 x uint32");
        if (!items.empty()) std::memcpy(items_out, items.data(), items.size() * sizeof(WorkItem));
        std::memcpy(cta_begin_out, cta_begin.data(), cta_begin.size() * 4);
    }
    return (uint32_t)items.size();
}

uint32_t mf_decode_plan_build_host_clusters(const uint32_t *kv_lens_host, uint32_t batch, uint32_t n_kv_heads,
                                            uint32_t max_ctas, uint32_t max_cluster, uint32_t clusters_of_16,
                                            uint32_t clusters_of_8, uint32_t *items_out, uint32_t item_capacity,
                                            uint32_t *n_ranges_out, uint32_t *cluster_out)
{
    if (!kv_lens_host || max_ctas == 0 || n_kv_heads == 0) return 0;
    std::vector<WorkItem> items;
    std::vector<uint32_t> cta_begin;
    uint32_t n_units = 0, cluster = (max_cluster & 0xFFu) | ((clusters_of_16 & 0xFFu) << 8) | ((clusters_of_8 & 0xFFu) << 16);
    uint64_t total = 0;
    build_decode_plan(kv_lens_host, batch, n_kv_heads, max_ctas, items, cta_begin, &n_units, &total, &cluster);
    if (n_ranges_out) *n_ranges_out = (uint32_t)cta_begin.size() - 1;
    if (cluster_out) *cluster_out = cluster;
    if (items.size() <= item_capacity && items_out && !items.empty()) std::memcpy(items_out, items.data(), items.size() * sizeof(WorkItem));
    return (uint32_t)items.size();
}

uint32_t mf_decode_plan_ctas(const MfDecodePlan *pl) { return pl ? pl->n_ctas : 0; }
uint32_t mf_decode_plan_cluster(const MfDecodePlan *pl) { return pl ? pl->cluster : 0; }
uint32_t mf_decode_plan_items(const MfDecodePlan *pl) { return pl ? pl->n_items : 0; }
uint64_t mf_decode_plan_tiles(const MfDecodePlan *pl) { return pl ? pl->total_tiles : 0; }

}  // extern "C"

namespace mf {

// Sequence-sharded decode: where this call's partials go in every rank's receive block, what it counts, waits for
// and merges (step parity, counted or tagged form).  Shared by the f16 and the 8-bit launchers.
mf_status setup_push(MfContext *ctx, const MfPeerExchange *px, uint32_t step, uint32_t merge_mask, uint64_t rows_in_call,
                     uint32_t D, DecodeParams &p)
{
    if (px->world == 0 || px->world > 8 || px->rank >= px->world)
        return fail(ctx, MF_ERR_INVALID_OPERATION, "peer exchange: rank %u of %u", px->rank, px->world);
    const uint64_t block = rows_in_call * (D + 2);
    p.push_world = px->world;
    for (uint32_t r = 0; r < px->world; ++r) {
        if (!px->recv[r] || !px->counters[r]) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "peer exchange: rank %u buffers", r);
        p.push_dst[r] = px->recv[r] + ((uint64_t)(step & 1) * px->world + px->rank) * block;
        p.push_cnt[r] = px->counters[r] + px->rank;
        p.push_unit_cnt[r] = px->counters[r] + kPeerUnitCounters;
    }
    // ranks that only merge: their merge of step - 2 read the parity block this step overwrites
    if (px->merge_only_mask >> px->rank & 1u)
        return fail(ctx, MF_ERR_INVALID_OPERATION, "peer exchange: rank %u is in merge_only_mask and cannot push", px->rank);
    if (px->merge_only_mask && step >= 2) {
        p.push_wait_mask = px->merge_only_mask & ((1u << px->world) - 1u);
        p.push_wait_expected = px->rows * (step - 1);
        p.push_merged_local = px->counters[px->rank] + kPeerMergedBy;
    }
    if (rows_in_call != px->rows || D != px->head_dim)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "peer exchange was created for %u rows x %u, this call has %llu x %u",
                    px->rows, px->head_dim, (unsigned long long)rows_in_call, D);
    if (merge_mask) {
        if (!(merge_mask >> px->rank & 1u) || (merge_mask >> px->world))
            return fail(ctx, MF_ERR_INVALID_OPERATION, "pusher mask 0x%x does not fit rank %u of %u", merge_mask, px->rank,
                        px->world);
        p.push_merge = 1;
        p.push_mask = merge_mask;
        p.push_expected = (uint32_t)__builtin_popcount(merge_mask) * (step + 1);
        p.push_local = px->recv[px->rank] + (uint64_t)(step & 1) * px->world * block;
        p.push_local_cnt = px->counters[px->rank] + kPeerUnitCounters;
        if (ctx->push_tagged && px->merge_only_mask == 0) {
            // tagged words: the same blocks, eight bytes per value, in a region of their own behind the plain
            // floats (a float left by a step in the counted form can then never be read as a tag)
            p.push_tagged = 1;
            p.push_tag = step + 1;
            const uint64_t tagged_base = (uint64_t)2 * px->world * block;
            for (uint32_t r = 0; r < px->world; ++r)
                p.push_dst[r] = px->recv[r] + tagged_base + 2 * (((uint64_t)(step & 1) * px->world + px->rank) * block);
            p.push_local = px->recv[px->rank] + tagged_base + 2 * ((uint64_t)(step & 1) * px->world * block);
        }
    }
    return MF_OK;
}

}  // namespace mf

extern "C" {

static mf_status paged_decode_common(MfContext *ctx, const MfDecodePlan *pl, const MfPagedKv *c,
                                     const MfPagedDecodeArgs *a, const uint32_t *rope_positions, float *acc, float *m,
                                     float *l, const MfPeerExchange *px = nullptr, uint32_t step = 0,
                                     uint32_t merge_mask = 0)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!pl || !c || !a) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged decode: null argument");
    if (!c->k_pool || !c->v_pool || !c->page_table || !c->kv_lens || !a->q)
        return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged decode: null tensor");
    if (!acc && !a->out && !(px && !merge_mask)) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged decode: output");
    if (a->append && (!a->k || !a->v)) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged decode: k/v of the new token");
    if (a->rope && (!a->cos || !a->sin)) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged decode: cos/sin");
    if (a->rope_mode > 1) return fail(ctx, MF_ERR_INVALID_OPERATION, "paged decode: rope_mode %u", a->rope_mode);
    if (c->batch != pl->batch || c->n_kv_heads != pl->n_kv_heads || c->head_dim != pl->head_dim ||
        a->n_heads != pl->n_heads || c->page_size != pl->page_size)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "paged decode: cache geometry differs from the plan");
    const uint32_t P = c->page_size;
    if (P < 8 || P > 256 || (P & (P - 1)) != 0)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "paged decode: page_size %u (power of two in 8..256)", P);
    if ((uint64_t)c->n_pages * c->n_kv_heads * P > 0x7FFFFFFFull)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "paged decode: pool has too many rows");
    if (pl->n_items == 0) return MF_OK;
    const uint32_t D = c->head_dim;
    DecodeParams p{};
    p.q = static_cast<const __half *>(a->q);
    p.k_new = static_cast<const __half *>(a->k);
    p.v_new = static_cast<const __half *>(a->v);
    p.q_rot = static_cast<__half *>(a->q_rot);
    p.out = static_cast<__half *>(a->out);
    p.cos_t = static_cast<const __half *>(a->cos);
    p.sin_t = static_cast<const __half *>(a->sin);
    p.k_base = static_cast<__half *>(c->k_pool);
    p.v_base = static_cast<__half *>(c->v_pool);
    p.page_table = c->page_table;
    p.kv_lens = c->kv_lens;
    p.rope_positions = rope_positions;
    p.items = pl->d_items;
    p.cta_item_begin = pl->d_cta_begin;
    p.cluster_size = pl->cluster;
    p.part_acc = pl->d_part_acc;
    p.part_ml = pl->d_part_ml;
    p.counters = pl->d_counters;
    p.out_acc = acc;
    p.out_m = m;
    p.out_l = l;
    p.status = ctx->d_status;
    p.n_heads = a->n_heads;
    p.n_kv_heads = c->n_kv_heads;
    p.group = a->n_heads / c->n_kv_heads;
    p.page_size = P;
    p.pt_stride = c->page_table_stride;
    p.n_pages = c->n_pages;
    p.batch = c->batch;
    p.rope = a->rope;
    p.rope_mode = a->rope_mode;
    p.append = a->append;
    p.q_stride_b = a->n_heads * D;
    p.q_stride_h = D;
    p.out_stride_b = a->n_heads * D;
    p.out_stride_h = D;
    p.knew_stride_b = c->n_kv_heads * D;
    p.scale_log2 = a->scale * 1.4426950408889634f;
    // Streaming K/V ahead of the previous kernel's end is safe when nothing in flight writes these pools.
    // With the fused append this call is their only writer in this step; without it the caller says so
    // (option value 2).  Not when a launch that may still be in flight appended to these same pools (a
    // one-layer model, two calls in a row on one cache): its new rows may not have landed yet.
    p.early_stream = (((ctx->overlap_launches && a->append) || ctx->overlap_launches == 2) &&
                      ctx->may_stream_early(c->k_pool, c->v_pool)) ? 1u : 0u;
    if (px) {
        const mf_status pst = setup_push(ctx, px, step, merge_mask, (uint64_t)c->batch * a->n_heads, D, p);
        if (pst != MF_OK) return pst;
    }
    CUtensorMap tm_k, tm_v;
    const uint64_t rows = (uint64_t)c->n_pages * c->n_kv_heads * P;
    const uint32_t box_rows = std::min(P, kTileKeys);
    mf_status st;
    p.whole_rows = (D == 128);
    if (p.whole_rows && (get_tensor_map(ctx, c->k_pool, rows, D, box_rows, 64, &tm_k, 1) != MF_OK ||
                         get_tensor_map(ctx, c->v_pool, rows, D, box_rows, 64, &tm_v, 1) != MF_OK))
        p.whole_rows = 0;
    if (!p.whole_rows) {
        if ((st = get_tensor_map(ctx, c->k_pool, rows, D, box_rows, 64, &tm_k)) != MF_OK) return st;
        if ((st = get_tensor_map(ctx, c->v_pool, rows, D, box_rows, 64, &tm_v)) != MF_OK) return st;
    }
    return launch_decode(ctx, tm_k, tm_v, p, D, pl->n_ctas, a->append ? c->k_pool : nullptr, a->append ? c->v_pool : nullptr);
}

mf_status mf_paged_decode(MfContext *ctx, const MfDecodePlan *plan, const MfPagedKv *cache, const MfPagedDecodeArgs *args)
{
    return paged_decode_common(ctx, plan, cache, args, nullptr, nullptr, nullptr, nullptr);
}

mf_status mf_paged_prefill(MfContext *ctx, const MfPagedKv *cache, const MfPagedPrefillArgs *a)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!cache || !cache->k_pool || !cache->v_pool || !cache->page_table || !a || !a->q || !a->out)
        return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged prefill: null input");
    if (a->q_len == 0 || a->kv_len == 0) return MF_OK;
    if (a->n_heads == 0 || cache->n_kv_heads == 0 || a->n_heads % cache->n_kv_heads != 0)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "paged prefill: n_heads %u, n_kv_heads %u", a->n_heads, cache->n_kv_heads);
    SdpaPrefillSplitKParams pp{};
    SdpaPrefillParams &b = pp.base;
    const uint32_t D = cache->head_dim;
    b.kv_len = a->kv_len;
    b.head_dim = D;
    b.scale = a->scale;
    b.stride_k_s = D;
    b.stride_v_s = D;
    b.query_offset = a->query_offset;
    b.q_stride_h = a->q_stride_h;
    b.q_stride_m = a->q_stride_m;
    b.out_stride_h = a->out_stride_h;
    b.out_stride_m = a->out_stride_m;
    b.group_size = a->n_heads / cache->n_kv_heads;
    b.q_len = a->q_len;
    pp.n_heads = a->n_heads;
    pp.split_k = effective_prefill_split_k(ctx, a->kv_len, a->q_len, a->n_heads);
    return launch_prefill(ctx, a->q, nullptr, nullptr, a->out, pp, cache, a->seq);
}

uint64_t mf_paged_prefill_kv8_workspace_bytes(const MfPagedKv8 *cache, uint32_t kv_len)
{
    if (!cache) return 0;
    // K and V of one sequence as f16 [Hkv, kv_len, D], each rounded up to 256 bytes
    const uint64_t one = ((uint64_t)cache->n_kv_heads * kv_len * cache->head_dim * 2 + 255) & ~(uint64_t)255;
    return 2 * one;
}

mf_status mf_paged_prefill_kv8(MfContext *ctx, const MfPagedKv8 *cache, const MfPagedPrefillArgs *a, void *workspace,
                               uint64_t workspace_bytes)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!cache || !a || !a->q || !a->out) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged prefill (8-bit): null input");
    if (a->q_len == 0 || a->kv_len == 0) return MF_OK;
    if (a->n_heads == 0 || cache->n_kv_heads == 0 || a->n_heads % cache->n_kv_heads != 0)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "paged prefill (8-bit): n_heads %u, n_kv_heads %u", a->n_heads, cache->n_kv_heads);
    const uint64_t need = mf_paged_prefill_kv8_workspace_bytes(cache, a->kv_len);
    if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return fail(ctx, MF_ERR_INVALID_OPERATION, "paged prefill (8-bit): workspace of %llu bytes, 256-byte aligned, needed",
                    (unsigned long long)need);
    // The sequence's rows, dequantised (e4m3 * row scale, rounded to f16), as a contiguous cache; then the f16 kernels.
    __half *kf = static_cast<__half *>(workspace);
    __half *vf = reinterpret_cast<__half *>(static_cast<char *>(workspace) + need / 2);
    mf_status st = mf_paged_kv8_gather(ctx, cache, 0, a->seq, a->kv_len, kf);
    if (st != MF_OK) return st;
    if ((st = mf_paged_kv8_gather(ctx, cache, 1, a->seq, a->kv_len, vf)) != MF_OK) return st;
    SdpaPrefillSplitKParams pp{};
    SdpaPrefillParams &b = pp.base;
    const uint32_t D = cache->head_dim;
    b.kv_len = a->kv_len;
    b.head_dim = D;
    b.scale = a->scale;
    b.stride_k_s = D;
    b.stride_v_s = D;
    b.k_stride_h = a->kv_len * D;
    b.v_stride_h = a->kv_len * D;
    b.query_offset = a->query_offset;
    b.q_stride_h = a->q_stride_h;
    b.q_stride_m = a->q_stride_m;
    b.out_stride_h = a->out_stride_h;
    b.out_stride_m = a->out_stride_m;
    b.group_size = a->n_heads / cache->n_kv_heads;
    b.q_len = a->q_len;
    pp.n_heads = a->n_heads;
    pp.split_k = effective_prefill_split_k(ctx, a->kv_len, a->q_len, a->n_heads);
    return launch_prefill(ctx, a->q, kf, vf, a->out, pp);
}

mf_status mf_paged_decode_partial_push(MfContext *ctx, const MfDecodePlan *plan, const MfPagedKv *cache,
                                       const MfPagedDecodeArgs *args, const uint32_t *rope_positions,
                                       const MfPeerExchange *px, uint32_t step)
{
    if (ctx && !px) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "peer exchange");
    return paged_decode_common(ctx, plan, cache, args, rope_positions, nullptr, nullptr, nullptr, px, step);
}

mf_status mf_paged_decode_push_merge(MfContext *ctx, const MfDecodePlan *plan, const MfPagedKv *cache,
                                     const MfPagedDecodeArgs *args, const uint32_t *rope_positions,
                                     const MfPeerExchange *px, uint32_t step, uint32_t pusher_mask)
{
    if (ctx && !px) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "peer exchange");
    if (ctx && !pusher_mask) return fail(ctx, MF_ERR_INVALID_OPERATION, "empty pusher mask");
    if (ctx && args && !args->out) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "push merge: output");
    return paged_decode_common(ctx, plan, cache, args, rope_positions, nullptr, nullptr, nullptr, px, step, pusher_mask);
}

mf_status mf_paged_decode_partial(MfContext *ctx, const MfDecodePlan *plan, const MfPagedKv *cache,
                                  const MfPagedDecodeArgs *args, const uint32_t *rope_positions, float *acc, float *m,
                                  float *l)
{
    if (ctx && (!acc || !m || !l)) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged decode partial: acc/m/l");
    return paged_decode_common(ctx, plan, cache, args, rope_positions, acc, m, l);
}

}  // extern "C"
