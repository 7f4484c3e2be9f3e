// Internal declarations shared by the translation units of libmetallic_cuda.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/metallic_cuda.h"

namespace mf {

constexpr uint32_t kTileKeys = 64;          // keys per pipeline stage
constexpr uint32_t kCounterRegionBytes = 64 * 1024;  // head of a scratch arena: unit counters
constexpr uint32_t kMaxUniformUnits = kCounterRegionBytes / 4;
// Bit of the device status word set when a kernel skipped a cache access because a page id taken
// from the caller's device-side table lies outside the pool, or a position outside the table
// (the lower bits record barrier waits that ran out).
constexpr uint32_t kStatusBadPage = 4096u;

// Word offsets inside a rank's peer-exchange counter block: per-source totals, "merged by rank" counts,
// per-unit arrival counters.
constexpr uint32_t kPeerMergedBy = 8;
constexpr uint32_t kPeerUnitCounters = 16;
constexpr uint32_t kStatusPushWait = 8192u;  // a pusher gave up waiting for a merge-only rank to free its block

// One span of KV tiles of one (sequence, kv head) unit, processed by one CTA.
struct WorkItem {
    uint32_t seq;
    uint32_t kvh;
    uint32_t tile_begin;
    uint32_t tile_end;
    uint32_t slot;        // partial slot written when the unit has several parts
    uint32_t unit;        // counter index
    uint32_t n_parts;     // number of items the unit was cut into
    uint32_t first_slot;  // slot of the unit's first part (parts are consecutive)
};

struct DecodeParams {
    const __half *q;
    const __half *k_new;
    const __half *v_new;
    __half *q_rot;
    __half *out;
    const __half *cos_t;
    const __half *sin_t;
    __half *k_base;
    __half *v_base;
    const uint32_t *page_table;
    const uint32_t *kv_lens;
    const uint32_t *rope_positions;
    const WorkItem *items;
    const uint32_t *cta_item_begin;
    float *part_acc;
    float *part_ml;
    uint32_t *counters;
    float *out_acc;
    float *out_m;
    float *out_l;
    uint32_t *status;
    uint32_t n_heads, n_kv_heads, group, page_size, pt_stride, batch;
    uint32_t n_pages;        // paged: pages in the pool (page ids are checked against it before a store)
    uint32_t k_rows_b, k_rows_h, v_rows_b, v_rows_h;  // contiguous: row strides
    uint32_t uniform_kv_len, uniform_tiles, uniform_span, uniform_total;
    uint32_t uniform_parts;  // > 0: every unit is cut into this many ranges of uniform_span tiles, one CTA each
    // Cluster form (short launches): a work item is processed by a thread-block cluster of `cluster_size`
    // CTAs, each taking an equal share of the item's tiles; the cluster combines its CTAs' states through
    // distributed shared memory and behaves as one CTA towards the rest (output, partial slot, ticket).
    // Item of cluster c: items[c] (explicit plan) or, for equal lengths, range c % uniform_parts of unit
    // c / uniform_parts.  0 or 1 = off.
    uint32_t cluster_size;
    uint32_t rope, rope_mode, append;
    uint32_t rope_position;  // contiguous mode: position of the query token
    uint32_t q_stride_b, q_stride_h, out_stride_b, out_stride_h;
    uint32_t knew_stride_b;  // elements between sequences in k_new / v_new
    uint32_t whole_rows;     // 1: one TMA box per page fetches both halves (3-D tensor map)
    uint32_t early_stream;   // 1: the producer may stream K/V before the previous kernel has finished
    uint32_t strict_release; // 1: dependents are released after this grid's own dependency wait, not at its start
    uint32_t release_late;   // 1: dependents are released when the producer has requested its last tile
    // Push mode (sequence-sharded decode): the finished (acc, m, l) of every unit is stored straight
    // into each rank's receive block over NVLink and announced on that rank's arrival counter.
    uint32_t push_world;     // 0 = off
    float *push_dst[8];      // rank r's receive block for THIS rank and step parity, as mapped here
    uint32_t *push_cnt[8];   // rank r's arrival counter for THIS rank
    uint32_t *push_unit_cnt[8];  // rank r's per-unit arrival counters
    // Merge inside the kernel: after pushing a unit, wait for the ranks of push_mask and write `out`.
    // Tagged words: every float travels with the step's tag in one 8-byte store, so a reader trusts a word as soon as
    // it carries the tag: no system-scope fence, no arrival counters (only with push_merge and no merge-only ranks).
    uint32_t push_tagged, push_tag;
    uint32_t push_merge;     // 0 = the caller merges with a second kernel
    uint32_t push_mask;      // ranks that push in this step
    uint32_t push_expected;  // value the unit counter reaches when all of them have
    const float *push_local; // this rank's receive blocks of this step parity: [world][block]
    const uint32_t *push_local_cnt;  // this rank's per-unit arrival counters
    // Back-pressure of ranks that only merge (they never wait for anybody, so nothing else keeps a pusher
    // from overwriting the parity block they still read): before this launch's first push, wait until every
    // rank of push_wait_mask has counted push_wait_expected merged rows on this rank's "merged by" words.
    uint32_t push_wait_mask;
    uint32_t push_wait_expected;
    const uint32_t *push_merged_local;
    float scale_log2;
};

// What a piece of a (sequence, kv head) unit costs the CTA that takes it, in tiles (q staging, combine, partial,
// ticket, and for one piece of a unit its merge: 5-10 us against 0.5-1.4 us per tile; 20 measured best for the f16 and
// the 8-bit cache alike), and the shortest piece worth that cost.  MF_OPTION_PLAN_ITEM_COST.
constexpr uint32_t kPlanItemCost = 20;
constexpr uint32_t kMinPieceTiles = 4;

struct TensorMapKey {
    const void *base;
    uint64_t rows;
    uint32_t cols;
    uint32_t box_rows;
    uint32_t box_cols;
    uint32_t whole_rows;  // 1: 3-D map whose box spans both 64-column halves of a row
    bool operator==(const TensorMapKey &o) const
    {
        return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows &&
               box_cols == o.box_cols && whole_rows == o.whole_rows;
    }
};
struct TensorMapKeyHash {
    size_t operator()(const TensorMapKey &k) const
    {
        uint64_t h = reinterpret_cast<uint64_t>(k.base) * 0x9E3779B97F4A7C15ull;
        h ^= k.rows + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
        h ^= (uint64_t(k.cols) << 32 | k.box_rows) + (h << 6) + (h >> 2);
        h ^= (k.box_cols * 2 + k.whole_rows) + (h << 6) + (h >> 2);
        return static_cast<size_t>(h);
    }
};

}  // namespace mf

struct MfContext {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    int sm_count = 0;
    std::string last_error;
    void *scratch = nullptr;
    uint64_t scratch_bytes = 0;
    bool scratch_owned = false;
    uint32_t *d_status = nullptr;
    uint64_t launches = 0;
    std::unordered_map<mf::TensorMapKey, CUtensorMap, mf::TensorMapKeyHash> tmaps;
    void *encode_fn = nullptr;
    // prefill_tc: the order in which the CTAs of the last launch shape take their (query tile, head) items
    uint32_t tc_order_key[6] = {0, 0, 0, 0, 0, 0};
    uint16_t tc_order[512];
    uint32_t tc_order_n = 0;
    uint32_t overlap_launches = 0;  // MF_OPTION_OVERLAP_LAUNCHES
    // Early K/V streaming under programmatic dependent launches, and what bounds it.
    //
    // A kernel launched with the programmatic attribute may start as soon as every CTA of the launch in
    // front of it has released its dependents (or exited).  Every such kernel of this library
    // (decode_kernel, fused_qkv_kernel, merge_pushed_kernel) takes a flag: RELAXED launches release at their
    // very start, STRICT launches only after their own dependency wait has returned - and that wait returns
    // only when the launch in front has completed, which in turn had waited for the one before it.
    // Claim: when launch m starts, every launch still in flight lies in {s, ..., m-1}, s being the last
    // strict launch before m.  (If m-1 is strict, all its CTAs saw m-2 complete before m could start.  If
    // m-1 is relaxed, m starting only shows that m-1 has started; whatever bound held at m-1's start still
    // holds, and s is the same for both.)  A launch made without the attribute starts after everything
    // before it has completed, so it can only shrink that set.
    // The context therefore keeps the caches written by the launches since the last strict one (at most
    // kWindow of them: every kWindow-th launch with the attribute is made strict) and a decode launch may
    // stream a cache ahead of its own wait only if that cache is not in the list.  The decision is exact in
    // the sense that it follows from the launch protocol alone, not from grid sizes or timing.
    static constexpr int kWindow = 8;
    const void *inflight_k[kWindow] = {}, *inflight_v[kWindow] = {};
    int n_inflight = 0;      // entries of the list
    int since_strict = 0;    // launches with the attribute after the last strict one
    bool may_stream_early(const void *k_cache, const void *v_cache) const
    {
        for (int i = 0; i < n_inflight; ++i)
            if (k_cache == inflight_k[i] || k_cache == inflight_v[i] || v_cache == inflight_k[i] || v_cache == inflight_v[i])
                return false;
        return true;
    }
    // Whether the next launch with the attribute has to be strict.
    bool next_launch_strict() const { return since_strict + 1 >= kWindow; }
    // After such a launch succeeded; k_cache / v_cache: what it writes (null: no cache).
    void note_programmatic_launch(bool strict, const void *k_cache, const void *v_cache)
    {
        if (strict) {
            n_inflight = 0;
            since_strict = 0;
        } else {
            ++since_strict;
        }
        if ((k_cache || v_cache) && n_inflight < kWindow) {
            inflight_k[n_inflight] = k_cache;
            inflight_v[n_inflight] = v_cache;
            ++n_inflight;
        }
    }
    uint32_t decode_stages = 0;     // MF_OPTION_DECODE_STAGES (0 = default)
    void *allgather_fn = nullptr;   // mf_context_set_allgather: replaces ncclAllGather in mf_allgather_merge
    uint32_t decode_clusters = 0;   // MF_OPTION_DECODE_CLUSTERS: 0 = the library decides, 1 = never
    uint32_t prefill_impl = 0;      // MF_OPTION_PREFILL_IMPL: 0 auto, 1 mma.sync, 2 tcgen05 only
    uint32_t plan_item_cost = mf::kPlanItemCost;  // MF_OPTION_PLAN_ITEM_COST
    uint32_t push_tagged = 1;       // MF_OPTION_PUSH_TAGGED: 1 = tagged words in the fused exchange, 0 = fence + counters
    uint32_t qkv_impl = 0;          // MF_OPTION_QKV_IMPL: 0 auto (tcgen05 from 8 input rows), 1 mma.sync, 2 tcgen05 whenever the shape allows
    void *qkv_xn = nullptr;         // normalised input rows of the tcgen05 projection
    size_t qkv_xn_bytes = 0;
};

struct MfDecodePlan {
    uint32_t batch = 0, n_heads = 0, n_kv_heads = 0, head_dim = 0, page_size = 0;
    uint32_t max_ctas = 0, n_ctas = 0, n_items = 0, n_units = 0;
    uint32_t cluster = 0, max_cluster = 0;  // cluster form of the current plan (0 = off) / what the device allows
    bool auto_ctas = false;           // the library picks the CTA count from the step's tile total
    uint32_t ctas_per_sm = 1, sm_count = 0;
    uint64_t total_tiles = 0;
    uint32_t item_capacity = 0;
    std::vector<mf::WorkItem> h_items;
    std::vector<uint32_t> h_cta_begin;
    // Two pinned staging sets used alternately, each guarded by the event recorded
    // after its upload, so that re-planning never has to drain the stream.
    mf::WorkItem *pinned_items[2] = {nullptr, nullptr};
    uint32_t *pinned_cta_begin[2] = {nullptr, nullptr};
    cudaEvent_t staged[2] = {nullptr, nullptr};
    uint32_t next_stage = 0;
    mf::WorkItem *d_items = nullptr;
    uint32_t *d_cta_begin = nullptr;
    float *d_part_acc = nullptr;
    float *d_part_ml = nullptr;
    uint32_t *d_counters = nullptr;
    uint32_t heads_padded = 0;
};

namespace mf {

mf_status fail(MfContext *ctx, mf_status code, const char *fmt, ...);
mf_status check_cuda(MfContext *ctx, cudaError_t e, const char *what);
mf_status check_launch(MfContext *ctx, const char *what);

// f16 tensor checks used by the operator entry points.
mf_status need_tensor(MfContext *ctx, const MfTensor *t, const char *name);
inline __half *tensor_ptr(const MfTensor *t)
{
    return reinterpret_cast<__half *>(static_cast<char *>(t->dev_ptr) + t->offset_bytes);
}

// Cached f16 tensor map over [rows, cols] with the 128-byte swizzle.  whole_rows == 0: 2-D map,
// box [box_rows, 64 cols].  whole_rows == 1 (cols == 128): 3-D map (64 cols, rows, 2 halves) whose
// box [64, box_rows, 2] brings whole 256-byte rows in one copy, laid out [half][box_rows][128 B].
mf_status get_tensor_map(MfContext *ctx, const void *base, uint64_t rows, uint32_t cols,
                         uint32_t box_rows, uint32_t box_cols, CUtensorMap *out,
                         uint32_t whole_rows = 0);

mf_status ensure_scratch(MfContext *ctx, uint64_t bytes);

// Host planner: cut the tiles of all (sequence, kv head) units into n_ctas equal spans.
// cluster_out (optional): in: the largest cluster allowed; out: the cluster size of the plan (0 = plain
// form).  In the cluster form there is one item per cluster and cta_begin is not used by the kernel.
void build_decode_plan(const uint32_t *kv_lens, uint32_t batch, uint32_t n_kv_heads,
                       uint32_t max_ctas, std::vector<WorkItem> &items,
                       std::vector<uint32_t> &cta_begin, uint32_t *n_units,
                       uint64_t *total_tiles, uint32_t *cluster_out = nullptr, uint32_t item_cost = kPlanItemCost);

// Resident decode CTAs per SM for a head_dim / GQA group size (decode.cu).
uint32_t decode_ctas_per_sm(const MfContext *ctx, uint32_t head_dim, uint32_t group);
// How a decode with equal lengths is cut: parts > 0 means every (sequence, kv head) unit is cut into
// `parts` ranges of `span` tiles, one CTA each (no CTA straddles two units); parts == 0 means equal
// spans over the flat tile list.
struct UniformSplit {
    uint32_t span, n_ctas, parts;
    uint32_t cluster;  // > 1: cluster form, `parts` ranges per unit, each processed by a cluster of this many CTAs
};
// max_cluster: largest cluster the launch may use (0 or 1: no cluster form).
UniformSplit uniform_split(uint32_t units, uint32_t tiles_per_unit, uint32_t n_splits, uint32_t want_ctas,
                           uint32_t max_cluster = 0);
// Largest cluster size (16, 8 or 0) the decode kernel for this head_dim / group can be launched with on the
// context's device; 0 when clusters are switched off.
uint32_t decode_max_cluster(MfContext *ctx, uint32_t head_dim, uint32_t group);
// Sequence-sharded decode: fills the exchange fields of a launch's parameters (attention_api.cu).
mf_status setup_push(MfContext *ctx, const MfPeerExchange *px, uint32_t step, uint32_t merge_mask, uint64_t rows_in_call,
                     uint32_t D, DecodeParams &p);
uint32_t decode_cta_target(uint32_t sm_count, uint32_t ctas_per_sm, uint64_t total_tiles);

// Launchers (decode.cu, prefill.cu, kv_append.cu).
// writes_k / writes_v: the caches this launch appends to (null when it only reads).
mf_status launch_decode(MfContext *ctx, const CUtensorMap &tm_k, const CUtensorMap &tm_v,
                        DecodeParams &p, uint32_t head_dim, uint32_t n_ctas, const void *writes_k = nullptr,
                        const void *writes_v = nullptr);

}  // namespace mf
