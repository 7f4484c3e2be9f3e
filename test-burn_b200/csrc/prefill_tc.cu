// Causal chunked prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM),
// head_dim 64 or 128, for query chunks of 64 rows or more.
//
// Same contract as prefill.cu (flash_prefill.metal:94-446 of the reference): key k is
// visible to query row r iff k <= r + query_offset, f16 x f16 products accumulated in f32,
// `scale`, running max from -1e30, f32 weights / l / accumulator, acc * (1/l) or 0, rows past
// q_len not written.  P is rounded to f16 for the PV product.
//
// One CTA per (128-row query tile, query head), walking the visible 128-key tiles in order.
//   warps 0-3   softmax group 0 (even tiles), warps 4-7 group 1 (odd tiles); one thread per query
//               row (= TMEM lane) holds the row's 128 scores in registers: warp w works on lane
//               quadrant w % 4
//   warp 8      TMA producer: Q tile once, then rings of 128-key K and V tiles (3 deep each)
//   warp 9      TMEM allocation and the single thread that issues tcgen05.mma
// Three score buffers and ONE output accumulator live in TMEM.  Per tile i, buffer b = i % 3:
//   S_b = Q K_i^T (A, B from 128-byte-swizzled shared memory, accumulator in TMEM)
//   -> group i % 2 reads S_b with tcgen05.ld, folds the row maxima into the running reference
//      m_ref (handed between the groups through shared memory, a few hundred cycles per tile),
//      writes P (f16) over the first 64 columns of S_b with tcgen05.st
//   -> O += P V_i (A from TMEM, B = V tile as an MN-major operand), O staying in TMEM
//   -> Q K_{i+3}^T is issued behind that product into the same buffer.
// With three buffers the two groups exponentiate two tiles at once while the tensor pipe works
// on the third.  O is only rescaled when a row's maximum has grown by more than 2^8 since the
// last rescale (the weights are then at most 256, which f16 holds without loss of relative
// precision); the final normalisation uses the reference maximum actually applied.
//
// TMEM columns (512): S_0/P_0 [0,128)  S_1/P_1 [128,256)  S_2/P_2 [256,384)  O [384,512).
#include <algorithm>
#include <cstring>
#include <queue>
#include <vector>

#include "internal.hpp"
#include "ptx.cuh"
#include "tcgen05.cuh"

namespace mf {
namespace {

constexpr uint32_t kBM = 128;             // query rows per CTA
constexpr uint32_t kBN = 128;             // keys per tile
constexpr uint32_t kRowSplit = 1;                         // softmax threads per query row
constexpr uint32_t kCols = 128 / kRowSplit;               // score columns per thread
constexpr uint32_t kGroupWarps = 4 * kRowSplit;           // softmax warps per group
constexpr uint32_t kSoftmaxWarps = 2 * kGroupWarps;
constexpr uint32_t kSoftmaxThreads = 32 * kSoftmaxWarps;
constexpr uint32_t kTcThreads = kSoftmaxThreads + 96;
constexpr float kRescaleThreshold = 8.0f;                 // log2 of the largest weight kept in P
constexpr uint32_t kHalfTile = 128 * 128; // bytes: 128 rows x 64 f16
__host__ __device__ constexpr uint32_t tc_tile_bytes(uint32_t d) { return (d / 64) * kHalfTile; }  // 16 or 32 KB
constexpr uint32_t kKStages = 3;           // K tiles in flight
constexpr uint32_t kVStages = 3;  // V tiles in flight
constexpr uint64_t kTcWaitNs = 2000000000ull;
constexpr float kNegInf = -1e30f;

struct TcParams {
    __half *out;
    uint32_t *status;
    uint32_t q_len, kv_len, query_offset, group, n_heads, n_q_tiles;
    // The (query tile << 8 | head) item of every CTA, in launch order (use_order; else the arithmetic longest-first order)
    uint32_t use_order;
    uint16_t order[512];
    uint32_t out_stride_h, out_stride_m;
    float scale_log2;
    // paged cache: K/V tiles are gathered page by page through the sequence's page-table row
    const uint32_t *page_table_row;  // null: contiguous cache
    uint32_t page_size, page_shift, n_kv_heads;  // page_size = 1 << page_shift
};

// Instruction descriptor of this kernel's products: M = 128.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t n, uint32_t b_mn_major)
{
    return instr_desc_f16(kBM, n, b_mn_major);
}

__device__ __forceinline__ float max3(float a, float b, float c)
{
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// 4-D tiled load without a cache hint: (column in half, row, half, head).
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void *tmap, int32_t x, int32_t y, int32_t z, int32_t w,
                                            uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
        ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar)
        : "memory");
}

// Zero rows [first_dead, 128) of a V tile laid out [column half][128 rows][128 bytes]; called by the
// 128 * kRowSplit threads of one softmax group (rarely: kept out of line, off the tile loop's registers).
template <uint32_t D>
__device__ __noinline__ void clear_dead_rows(uint8_t *v_tile, uint32_t first_dead, uint32_t gtid, uint32_t page_shift)
{
    // paged V tile: [page][half][P rows][128 bytes] (head_dim 128), [128 rows][128 bytes] (head_dim 64)
    for (uint32_t c = gtid; c < (kBN - first_dead) * (D / 8); c += 128 * kRowSplit) {
        const uint32_t r = first_dead + c / (D / 8), ch = c % (D / 8);
        const uint32_t off = D == 64 ? r * 128
                                     : ((r >> page_shift) << (page_shift + 8)) + ((ch / 8) << (page_shift + 7)) +
                                           ((r & ((1u << page_shift) - 1)) << 7);
        *reinterpret_cast<uint4 *>(v_tile + off + (ch % 8) * 16) = make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async();
}

// Where the 16 keys of P V step kk start inside a V tile, and the distance between the two 64-column
// halves.  Contiguous cache (and head_dim 64): [half][128 rows][128 bytes].  Paged cache, head_dim 128:
// [page][half][P rows][128 bytes], one TMA copy per page.
template <uint32_t D, bool PAGED>
__device__ __forceinline__ uint32_t v_step_offset(uint32_t kk, uint32_t page_shift)
{
    if (!PAGED || D == 64) return kk * 2048;
    const uint32_t row = kk * 16;
    return ((row >> page_shift) << (page_shift + 8)) + ((row & ((1u << page_shift) - 1)) << 7);
}
template <uint32_t D, bool PAGED>
__device__ __forceinline__ uint32_t v_half_stride(uint32_t page_shift)
{
    return (!PAGED || D == 64) ? kHalfTile : (128u << page_shift);
}

// Distance between the two 8-key groups of a step: the next 1024 bytes, except with 8-row pages, where
// the second group is the next page.
template <uint32_t D, bool PAGED>
__device__ __forceinline__ uint32_t v_group_stride(uint32_t page_shift)
{
    return (PAGED && D == 128 && page_shift == 3) ? 2048u : 1024u;
}

// Barrier slots (8 bytes each) after the tiles.
enum Bar : uint32_t {
    kQFull = 0,
    kKFull = 1,    // [3] the first three K tiles
    kVFull = 4,    // [3] V tile i together with K tile i + 3
    kUnused7 = 7,  // [6] slots kept so that the numbering stays put
    kSFull = 13,   // [3] per score buffer: it holds Q K^T of its next tile
    kPFull = 16,   // [3] per score buffer: P is in it (and O has been rescaled if needed)
    kOFull = 19,   // [3] per score buffer: the P V that read it has completed
    kDec = 22,     // [2] by tile parity: the tile's row maxima have been folded into m_ref
    kNumBars = 24
};
static_assert(kKStages == 3 && kVStages == 3, "ring slot = score buffer = tile % 3");

__host__ __device__ constexpr uint32_t tc_smem_tiles(uint32_t d) { return tc_tile_bytes(d) * (1 + kKStages + kVStages); }  // Q + K ring + V ring
constexpr uint32_t kRefBytes = 128 * 4;                             // m_ref per query row
constexpr uint32_t kXmaxBytes = 0;
constexpr uint32_t kPidTiles = 8;                                   // page ids kept for this many tiles
constexpr uint32_t kPidBytes = kPidTiles * 32 * 4;                  // one id per producer lane and tile
__host__ __device__ constexpr uint32_t tc_smem_bytes(uint32_t d)
{
    return tc_smem_tiles(d) + kRefBytes + kXmaxBytes + kNumBars * 8 + 16 + kPidBytes + 1024;
}
static_assert(tc_smem_bytes(128) <= 227 * 1024, "shared memory");

// PAGED: K/V tiles gathered page by page (a separate instantiation: the extra code costs the
// contiguous form 3 % when it is merely present).
template <uint32_t D, bool PAGED>
__global__ void __launch_bounds__(kTcThreads, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const TcParams p)
{
    static_assert(D == 64 || D == 128, "head_dim");
    constexpr uint32_t kTile = tc_tile_bytes(D);             // one Q, K or V tile: 128 rows x D f16
    constexpr uint32_t kSmemTiles = tc_smem_tiles(D);
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t q_smem = smem_base;
    const uint32_t k_smem = smem_base + kTile;
    const uint32_t v_smem = k_smem + kKStages * kTile;
    volatile float *mref = reinterpret_cast<volatile float *>(smem + kSmemTiles);
    float *lbuf = reinterpret_cast<float *>(smem);  // epilogue only: the Q tile is no longer read
    const uint32_t bars = smem_base + kSmemTiles + kRefBytes + kXmaxBytes;
    volatile uint32_t *tmem_slot =
        reinterpret_cast<volatile uint32_t *>(smem + kSmemTiles + kRefBytes + kXmaxBytes + kNumBars * 8);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    auto bar = [&](uint32_t i) { return bars + i * 8; };

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // CTAs are handed out in blockIdx order.  Small grids come with the host's list (tc_item_order); else all heads
    // of the last (longest) query tile first, so that the short tiles fill the tail of the grid.
    const uint32_t q_tile = p.use_order ? p.order[blockIdx.x] >> 8 : p.n_q_tiles - 1 - blockIdx.x / p.n_heads;
    const uint32_t head = p.use_order ? p.order[blockIdx.x] & 0xFFu : blockIdx.x % p.n_heads;
    const uint32_t kvh = head / p.group;
    const uint32_t row0 = q_tile * kBM;
    const uint32_t last_row = min(p.q_len, row0 + kBM) - 1;
    const uint32_t key_end = min(p.kv_len, last_row + p.query_offset + 1);
    const uint32_t n_tiles = (key_end + kBN - 1) / kBN;

    if (tid == 0) {
        mbar_init(bar(kQFull), 1);
        for (uint32_t s = 0; s < 3; ++s) {
            mbar_init(bar(kKFull + s), 1);
            mbar_init(bar(kVFull + s), 1);
            mbar_init(bar(kSFull + s), 1);
            mbar_init(bar(kPFull + s), kGroupWarps);  // one arrival per softmax warp of the group
            mbar_init(bar(kOFull + s), 1);
        }
        mbar_init(bar(kDec), kGroupWarps);
        mbar_init(bar(kDec + 1), kGroupWarps);
        *abort_flag = 0;
        mbar_fence_init();
        fence_proxy_async();
    }
    if (warp == kSoftmaxWarps + 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // The common case is a barrier that has already completed: one try, nothing else.  (The thread that
    // issues the MMAs runs every instruction of this on the kernel's critical path.)
    auto wait = [&](uint32_t b, uint32_t parity, uint32_t code) {
        if (mbar_try_wait(b, parity)) return;
        if (!*abort_flag && !mbar_wait_bounded(b, parity, kTcWaitNs)) {
            *abort_flag = 1;
            atomicOr(p.status, code);
        }
    };

    if (warp == kSoftmaxWarps && PAGED) {
        // ------------------------------------------------ TMA producer, paged cache (whole warp) ---
        // A tile is 128 / P pages; lane l brings (page l / halves, column half l % halves) of a tile with
        // one copy of P rows x 128 bytes, to where the whole-tile box of the contiguous form would
        // have put those rows (P is a multiple of 8, so the 128-byte swizzle pattern lines up).  Page
        // ids are read six tiles ahead and parked in shared memory, one word per lane and tile.
        // Rows past kv_len are not loaded: K columns there are masked, V rows are cleared by the
        // softmax group of the last tile.
        constexpr uint32_t kHalves = D / 64, kHalfBytes = kBN * 128;
        const uint32_t P = p.page_size, per_tile = kBN / P;
        const uint32_t my_page = lane / kHalves, my_half = lane % kHalves;
        const uint32_t total_pages = (p.kv_len + P - 1) / P;
        uint32_t *pid = reinterpret_cast<uint32_t *>(smem + kSmemTiles + kRefBytes + kXmaxBytes + kNumBars * 8 + 16);
        auto pages_of = [&](uint32_t t) { return min(per_tile, total_pages - min(total_pages, t * per_tile)); };
        auto read_id = [&](uint32_t t) -> uint32_t {
            return (t < n_tiles && my_page < pages_of(t)) ? __ldg(p.page_table_row + t * per_tile + my_page) : 0u;
        };
        auto load_tile = [&](uint32_t dst_tile, const CUtensorMap *tm, uint32_t t, uint32_t barrier) {
            if (my_page < pages_of(t)) {
                const uint32_t id = pid[(t % kPidTiles) * 32 + lane];
                tma_load_4d(dst_tile + my_half * kHalfBytes + my_page * P * 128, tm, 0, 0, (int32_t)my_half,
                            (int32_t)(id * p.n_kv_heads + kvh), barrier);
            }
        };
        auto tile_bytes = [&](uint32_t t) { return pages_of(t) * P * D * 2; };
        for (uint32_t t = 0; t < 6; ++t) pid[(t % kPidTiles) * 32 + lane] = read_id(t);
        uint32_t pending = read_id(6);
        if (lane == 0) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_v);
            mbar_arrive_expect_tx(bar(kQFull), kTile);
            tma_load_4d(q_smem, &tm_q, 0, (int32_t)row0, 0, (int32_t)head, bar(kQFull));
            for (uint32_t i = 0; i < min(n_tiles, 3u); ++i) mbar_arrive_expect_tx(bar(kKFull + i), tile_bytes(i));
        }
        __syncwarp();
        for (uint32_t i = 0; i < min(n_tiles, 3u); ++i) load_tile(k_smem + i * kTile, &tm_k, i, bar(kKFull + i));
        uint32_t b = 0, ph = 0;  // slot i % 3 and phase (i / 3) & 1
        for (uint32_t i = 0; i < n_tiles; ++i) {
            // ids of tile i + 6 arrived during the last iteration; those of tile i + 7 are requested now
            pid[((i + 6) % kPidTiles) * 32 + lane] = pending;
            pending = read_id(i + 7);
            const bool with_k = i + 3 < n_tiles;
            if (lane == 0) {
                if (i >= 3) wait(bar(kOFull + b), ph ^ 1, 16u);  // P V (i - 3) done: V slot b is free
                mbar_arrive_expect_tx(bar(kVFull + b), tile_bytes(i) + (with_k ? tile_bytes(i + 3) : 0u));
            }
            __syncwarp();
            // V: one copy per page, both column halves, landing as [page][half][P rows][128 bytes]; the
            // P V products address it with their own descriptor (see v_step_offsets).  The page's id
            // sits in the ring slot of the lane that brings the page's first K half.
            if (lane < pages_of(i))
                tma_load_4d(v_smem + b * kTile + lane * (kHalves * P * 128), &tm_v, 0, 0, 0,
                            (int32_t)(pid[(i % kPidTiles) * 32 + lane * kHalves] * p.n_kv_heads + kvh), bar(kVFull + b));
            if (with_k) {
                if (lane == 0) wait(bar(kSFull + b), ph, 16u);  // Q K^T (i) done: K slot b is free
                __syncwarp();
                load_tile(k_smem + b * kTile, &tm_k, i + 3, bar(kVFull + b));
            }
            if (++b == 3) {
                b = 0;
                ph ^= 1;
            }
        }
    } else if (warp == kSoftmaxWarps) {
        // ---------------------------------------------------------------- TMA producer ---
        if (lane == 0) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_v);
            mbar_arrive_expect_tx(bar(kQFull), kTile);
            tma_load_4d(q_smem, &tm_q, 0, (int32_t)row0, 0, (int32_t)head, bar(kQFull));
            // K/V maps are (head_dim, kv_len, kv heads): rows past kv_len arrive as zeros, so a
            // never-written cache row cannot meet a zero weight as NaN.
            // The first three K tiles have barriers of their own; after that V(i) and K(i + 3) travel as a
            // pair on ONE barrier, because the MMA-issuing thread wants them together (P V of tile i, then
            // Q K^T of tile i + 3) and every wait it makes is on the kernel's critical path.  The V slot
            // is free when the P V that read it has completed, the K slot when the Q K^T of tile i has:
            // the tensor pipe's own completion barriers say both.
            for (uint32_t i = 0; i < min(n_tiles, 3u); ++i) {
                mbar_arrive_expect_tx(bar(kKFull + i), kTile);
                tma_load_4d(k_smem + i * kTile, &tm_k, 0, (int32_t)(i * kBN), 0, (int32_t)kvh, bar(kKFull + i));
            }
            uint32_t b = 0, ph = 0;  // slot i % 3 and phase (i / 3) & 1
            for (uint32_t i = 0; i < n_tiles; ++i) {
                if (i >= 3) { wait(bar(kOFull + b), ph ^ 1, 16u); }  // P V (i - 3) done
                const bool with_k = i + 3 < n_tiles;
                mbar_arrive_expect_tx(bar(kVFull + b), (with_k ? 2 : 1) * kTile);
                tma_load_4d(v_smem + b * kTile, &tm_v, 0, (int32_t)(i * kBN), 0, (int32_t)kvh, bar(kVFull + b));
                if (with_k) {
                    wait(bar(kSFull + b), ph, 16u);  // Q K^T (i) done: K slot b is free
                    tma_load_4d(k_smem + b * kTile, &tm_k, 0, (int32_t)((i + 3) * kBN), 0, (int32_t)kvh, bar(kVFull + b));
                }
                if (++b == 3) {
                    b = 0;
                    ph ^= 1;
                }
            }
        }
    } else if (warp == kSoftmaxWarps + 2) {
        // ------------------------------------------------ MMA issuer for Q K^T (split issue) ---
        if (lane == 0) {
            constexpr uint32_t kIdescQK = instr_desc(kBN, 0);
            wait(bar(kQFull), 0, 32u);
            const uint64_t q_desc = smem_desc(q_smem, 16, 1024);
            uint32_t b = 0, ph = 0;  // tile i: buffer i % 3, phase (i / 3) & 1
            for (uint32_t i = 0; i < n_tiles; ++i) {
                if (i < 3) {
                    wait(bar(kKFull + b), 0, 32u);
                } else {
                    wait(bar(kVFull + b), ph ^ 1, 32u);  // K(i) came with V(i - 3)
                    wait(bar(kOFull + b), ph ^ 1, 32u);  // P V (i - 3) has read the buffer
                }
                tc_fence_after();
                const uint64_t k_desc = smem_desc(k_smem + b * kTile, 16, 1024);
#pragma unroll
                for (uint32_t kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = ((kk >> 2) * kHalfTile + (kk & 3) * 32) >> 4;
                    tc_mma_ss(tmem + b * 128, q_desc + off, k_desc + off, kIdescQK, kk > 0);
                }
                tc_commit(bar(kSFull + b));
                if (++b == 3) {
                    b = 0;
                    ph ^= 1;
                }
            }
        }
    } else if (warp == kSoftmaxWarps + 1) {
        // ------------------------------------------------- MMA issuer for P V (split issue) ---
        if (lane == 0) {
            constexpr uint32_t kIdescPV = instr_desc(D, 1);
            uint32_t voff[kBN / 16];  // descriptor address steps of the eight products of a tile
#pragma unroll
            for (uint32_t kk = 0; kk < kBN / 16; ++kk) voff[kk] = v_step_offset<D, PAGED>(kk, p.page_shift) >> 4;
            uint32_t b = 0, ph = 0;
            for (uint32_t i = 0; i < n_tiles; ++i) {
                wait(bar(kVFull + b), ph, 64u);
                wait(bar(kPFull + b), ph, 64u);
                tc_fence_after();
                const uint64_t v_desc = smem_desc(v_smem + b * kTile, v_half_stride<D, PAGED>(p.page_shift), v_group_stride<D, PAGED>(p.page_shift));
#pragma unroll
                for (uint32_t kk = 0; kk < kBN / 16; ++kk)
                    tc_mma_ts(tmem + 384, tmem + b * 128 + kk * 8, v_desc + voff[kk], kIdescPV, (i > 0 || kk > 0) ? 1u : 0u);
                tc_commit(bar(kOFull + b));
                if (++b == 3) {
                    b = 0;
                    ph ^= 1;
                }
            }
        }
    } else {
        // --------------------------------------------------------- softmax groups / epilogue ---
        // kRowSplit threads per query row (= TMEM lane) and group, each holding 128 / kRowSplit scores of
        // the row in registers.  With two threads per row the halves of a row swap their maxima through
        // shared memory once per tile; between tiles the two groups hand the row's reference maximum to
        // each other the same way.
        const uint32_t g = warp / (4 * kRowSplit);              // group: tiles i = g, g + 2, ...
        const uint32_t quad = warp & 3;
        const uint32_t half = (warp >> 2) % kRowSplit;          // which part of the row's columns
        const uint32_t r_in = quad * 32 + lane;                 // row inside the tile = TMEM lane
        const uint32_t row = row0 + r_in;
        const uint32_t lane_base = (quad * 32u) << 16;          // TMEM lane quadrant of this warp
        const uint32_t limit = row + p.query_offset;            // last visible key
        const uint32_t o_tm = tmem + lane_base + 384;
        const uint32_t last_ok = min(limit, p.kv_len - 1);
        const uint32_t col0 = half * kCols;                     // this thread's S columns
        const uint32_t pair_bar = 1 + g * 4 + quad;             // named barrier of the warps that share rows
        float my_ref = kNegInf, l_part = 0.f;                   // my_ref in the scaled log2 domain
        uint32_t last_mine = 0xFFFFFFFFu;

        for (uint32_t i = g; i < n_tiles; i += 2) {
            const uint32_t b = i % 3, sph = (i / 3) & 1;
            const uint32_t s_tm = tmem + lane_base + b * 128;   // S / P buffer of this tile
            const uint32_t key0 = i * kBN + col0;
            // Only tiles on the causal diagonal or at the end of the cache need a mask.
            const uint32_t n_vis = last_ok < key0 ? 0u : min(kCols, last_ok - key0 + 1);
            last_mine = i;
            wait(bar(kSFull + b), sph, 256u);
            tc_fence_after();
            // The TMEM accesses below are warp-collective: the choice between the plain and the
            // masked form of the row must be the same for all 32 rows of the warp.
            const bool whole = __all_sync(0xffffffffu, n_vis == kCols);
            float mx0 = -3.0e38f, mx1 = -3.0e38f, mx2 = -3.0e38f, mx3 = -3.0e38f;
            if (kRowSplit == 2) {
                // The row maximum needs the partner's columns too: stream them through registers for the
                // maximum only (cheaper than swapping maxima through shared memory, and exact).  Their
                // visible count follows from the same limit.
                const uint32_t pcol0 = (half ^ 1) * kCols;
                const uint32_t pkey0 = i * kBN + pcol0;
                const uint32_t p_vis = last_ok < pkey0 ? 0u : min(kCols, last_ok - pkey0 + 1);
                const bool p_whole = __all_sync(0xffffffffu, p_vis == kCols);
#pragma unroll
                for (uint32_t c = 0; c < kCols / 32; ++c) {
                    uint32_t t[32];
                    tmem_ld32(s_tm + pcol0 + c * 32, t);
                    tc_wait_ld();
                    if (p_whole) {
#pragma unroll
                        for (uint32_t q = 0; q < 32; q += 8) {
                            mx0 = max3(mx0, __uint_as_float(t[q]), __uint_as_float(t[q + 1]));
                            mx1 = max3(mx1, __uint_as_float(t[q + 2]), __uint_as_float(t[q + 3]));
                            mx2 = max3(mx2, __uint_as_float(t[q + 4]), __uint_as_float(t[q + 5]));
                            mx3 = max3(mx3, __uint_as_float(t[q + 6]), __uint_as_float(t[q + 7]));
                        }
                    } else {
#pragma unroll
                        for (uint32_t q = 0; q < 32; ++q)
                            if (c * 32 + q < p_vis) mx0 = fmaxf(mx0, __uint_as_float(t[q]));
                    }
                }
            }
            uint32_t r[kCols];
#pragma unroll
            for (uint32_t c = 0; c < kCols / 32; ++c)
                tmem_ld32(s_tm + col0 + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
            tc_wait_ld();
            // row maximum of the raw scores (the scale is positive)
            if (whole) {
#pragma unroll
                for (uint32_t q = 0; q < kCols; q += 8) {
                    mx0 = max3(mx0, __uint_as_float(r[q]), __uint_as_float(r[q + 1]));
                    mx1 = max3(mx1, __uint_as_float(r[q + 2]), __uint_as_float(r[q + 3]));
                    mx2 = max3(mx2, __uint_as_float(r[q + 4]), __uint_as_float(r[q + 5]));
                    mx3 = max3(mx3, __uint_as_float(r[q + 6]), __uint_as_float(r[q + 7]));
                }
            } else {
#pragma unroll
                for (uint32_t q = 0; q < kCols; ++q) {
                    if (q >= n_vis) r[q] = 0xFF800000u;  // -inf: weight exactly 0 below
                    mx0 = fmaxf(mx0, __uint_as_float(r[q]));
                }
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            if (kRowSplit == 2) {
                // Both threads of a row have every score they need in registers: from here on either may
                // overwrite the buffer with P.
                named_bar_sync(pair_bar, 64);
            }
            const float m_new = mx > -3.0e38f ? mx * p.scale_log2 : kNegInf;
            // The reference maximum after tile i - 1, decided by the other group.
            float m_prev = kNegInf;
            if (i > 0) {
                wait(bar(kDec + ((i - 1) & 1)), ((i - 1) >> 1) & 1, 512u);
                m_prev = mref[r_in];
            }
            // Lazy rescale: keep exponentiating against the old reference until a row outgrows it by 2^8.
            const bool grow = m_new > m_prev + kRescaleThreshold;
            const float m_ref = grow ? m_new : m_prev;
            if (m_ref != my_ref) {
                l_part *= fast_exp2(my_ref - m_ref);
                my_ref = m_ref;
            }
            if (i > 0 && __any_sync(0xffffffffu, grow)) {
                // O must hold every earlier P V before it is scaled.  S(i) being there implies that
                // P V (i - 3) is done, so the parity of the buffer's barrier is unambiguous.
                const uint32_t pb = (i - 1) % 3;
                wait(bar(kOFull + pb), ((i - 1) / 3) & 1, 128u);
                tc_fence_after();
                const float alpha = fast_exp2(m_prev - m_ref);
#pragma unroll 1
                for (uint32_t c = 0; c < D / kRowSplit / 32; ++c) {  // this thread's share of the row's O columns
                    uint32_t ob[32];
                    tmem_ld32(o_tm + half * (D / kRowSplit) + c * 32, ob);
                    tc_wait_ld();
#pragma unroll
                    for (uint32_t q = 0; q < 32; ++q) ob[q] = __float_as_uint(__uint_as_float(ob[q]) * alpha);
                    tmem_st32(o_tm + half * (D / kRowSplit) + c * 32, ob);
                }
                tc_wait_st();
                // The scores are fetched again rather than kept in registers across this rare block.
#pragma unroll
                for (uint32_t c = 0; c < kCols / 32; ++c)
                    tmem_ld32(s_tm + col0 + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
                tc_wait_ld();
                if (!whole) {
#pragma unroll
                    for (uint32_t q = 0; q < kCols; ++q)
                        if (q >= n_vis) r[q] = 0xFF800000u;
                }
                // The partner warp holds the same rows, took the same decision and is in this block too:
                // neither may write P before both have their scores back.
                if (kRowSplit == 2) named_bar_sync(pair_bar, 64);
            }
            if (half == 0) mref[r_in] = m_ref;  // both threads of a row reach the same decision
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kDec + (i & 1)));  // the other group may fold in tile i + 1
            // weights (f16) over the first 64 columns of the buffer, and the row sum
            if (whole) {
                const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nm2 = make_float2(-m_ref, -m_ref);
                float2 acc_a = make_float2(0.f, 0.f), acc_b = make_float2(0.f, 0.f);
#pragma unroll
                for (uint32_t c = 0; c < kCols / 32; ++c) {
                    uint32_t pk[16];
#pragma unroll
                    for (uint32_t q = 0; q < 16; ++q) {
                        const float2 t = __ffma2_rn(make_float2(__uint_as_float(r[c * 32 + 2 * q]),
                                                                __uint_as_float(r[c * 32 + 2 * q + 1])), sc2, nm2);
                        float2 w;
                        w.x = fast_exp2(t.x);
                        w.y = fast_exp2(t.y);
                        if (q & 1) acc_b = __fadd2_rn(acc_b, w);
                        else acc_a = __fadd2_rn(acc_a, w);
                        pk[q] = pack_f16x2(w.x, w.y);
                    }
                    tmem_st16(s_tm + col0 / 2 + c * 16, pk);
                }
                const float2 acc = __fadd2_rn(acc_a, acc_b);
                l_part += acc.x + acc.y;  // relative to my_ref
            } else {
                float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
                for (uint32_t c = 0; c < kCols / 32; ++c) {
                    uint32_t pk[16];
#pragma unroll
                    for (uint32_t q = 0; q < 16; ++q) {
                        const float p0 = fast_exp2(fmaf(__uint_as_float(r[c * 32 + 2 * q]), p.scale_log2, -m_ref));
                        const float p1 = fast_exp2(fmaf(__uint_as_float(r[c * 32 + 2 * q + 1]), p.scale_log2, -m_ref));
                        sum0 += p0;
                        sum1 += p1;
                        pk[q] = pack_f16x2(p0, p1);
                    }
                    tmem_st16(s_tm + col0 / 2 + c * 16, pk);
                }
                l_part += sum0 + sum1;
            }
            if (PAGED && i + 1 == n_tiles && p.kv_len < (i + 1) * kBN) {
                // Paged cache: the rows of this tile past kv_len were never written or never loaded.
                // Their weights are exactly zero, but zero times a stale NaN is not: clear them in V
                // once V(i) has landed and before this group reports P(i).
                wait(bar(kVFull + b), sph, 64u);
                clear_dead_rows<D>(smem + (v_smem - smem_base) + b * kTile, p.kv_len - i * kBN,
                                   (warp % (4 * kRowSplit)) * 32 + lane, p.page_shift);
            }
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kPFull + b));  // P(i) is in TMEM, O is consistent with m_ref
        }

        // ---- normalise and write the rows out: every thread takes 128 / (2 kRowSplit) columns --------
        if (last_mine != 0xFFFFFFFFu) {
            // The product of this group's last tile; the other group waits for its own, and both
            // issuing threads' products on O have then completed.
            wait(bar(kOFull + last_mine % 3), (last_mine / 3) & 1, 128u);
        }
        named_bar_sync(9, kSoftmaxThreads);  // every product is done, every decision published
        tc_fence_after();
        const float m_fin = mref[r_in];
        lbuf[(g * kRowSplit + half) * 128 + r_in] = l_part * fast_exp2(my_ref - m_fin);
        named_bar_sync(10, kSoftmaxThreads);
        float l_tot = 0.f;
#pragma unroll
        for (uint32_t s2 = 0; s2 < 2 * kRowSplit; ++s2) l_tot += lbuf[s2 * 128 + r_in];
        const float inv = ((fabsf(l_tot) <= 3.0e38f) && fabsf(l_tot) > 1e-6f) ? 1.0f / l_tot : 0.f;
        constexpr uint32_t kOutCols = D / (2 * kRowSplit);
        const uint32_t oc0 = (g * kRowSplit + half) * kOutCols;
        __half *dst = p.out + (size_t)row * p.out_stride_m + (size_t)head * p.out_stride_h + oc0;
#pragma unroll 1
        for (uint32_t c = 0; c < kOutCols / 32; ++c) {
            float o[32];
            tmem_ld32(o_tm + oc0 + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&o[0]));
            tc_wait_ld();
            if (row < p.q_len) {
#pragma unroll
                for (uint32_t d = 0; d < 32; d += 8) {
                    uint4 v;
                    v.x = pack_f16x2(o[d] * inv, o[d + 1] * inv);
                    v.y = pack_f16x2(o[d + 2] * inv, o[d + 3] * inv);
                    v.z = pack_f16x2(o[d + 4] * inv, o[d + 5] * inv);
                    v.w = pack_f16x2(o[d + 6] * inv, o[d + 7] * inv);
                    *reinterpret_cast<uint4 *>(dst + c * 32 + d) = v;
                }
            }
        }
    }

    // Everybody meets here before the TMEM columns go back, also after an abort.
    tc_fence_before();
    __syncthreads();
    if (warp == kSoftmaxWarps + 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// The order in which a grid's CTAs take their (query tile, head) items.  The hardware hands CTAs to the SMs in
// blockIdx order, one per SM here, so a launch is list scheduling of n_items jobs of (key tiles + a fixed cost) on
// the SMs, and with 2-3 jobs per SM the longest-first list ends 10-14 % above the mean (measured on the C4 shape: the
// list below is 3-5 % faster).  Assignment: longest first onto the least loaded SM, then moves and swaps off the most
// loaded SM while they lower it; list: all jobs by their start time in that assignment, which list scheduling then
// reproduces.  Heads of a query tile are interchangeable and are numbered as they come.
constexpr float kTcItemFixedCost = 7.3f;  // what a CTA costs beyond its key tiles, in key tiles (fill, drain, launch)

void tc_item_order(const TcParams &p, uint32_t n_sms, uint16_t *order)
{
    const uint32_t nq = p.n_q_tiles, H = p.n_heads, n = nq * H, m = std::min(n_sms, n);
    std::vector<float> size(nq);
    for (uint32_t i = 0; i < nq; ++i) {
        const uint32_t last_row = std::min(p.q_len, (i + 1) * kBM) - 1;
        const uint32_t key_end = std::min(p.kv_len, last_row + p.query_offset + 1);
        size[i] = (float)((key_end + kBN - 1) / kBN) + kTcItemFixedCost;
    }
    std::vector<uint32_t> cls(nq);  // query tiles, longest first
    for (uint32_t i = 0; i < nq; ++i) cls[i] = i;
    std::stable_sort(cls.begin(), cls.end(), [&](uint32_t a, uint32_t b) { return size[a] > size[b]; });
    std::vector<std::vector<uint32_t>> on(m);  // query tile of every job of an SM
    std::vector<float> load(m, 0.f);
    {
        typedef std::pair<float, uint32_t> Slot;
        std::priority_queue<Slot, std::vector<Slot>, std::greater<Slot>> free_at;
        for (uint32_t s = 0; s < m; ++s) free_at.push(Slot(0.f, s));
        for (uint32_t ci = 0; ci < nq; ++ci)
            for (uint32_t h = 0; h < H; ++h) {
                const Slot s = free_at.top();
                free_at.pop();
                on[s.second].push_back(cls[ci]);
                load[s.second] = s.first + size[cls[ci]];
                free_at.push(Slot(load[s.second], s.second));
            }
    }
    for (uint32_t round = 0; round < 512; ++round) {
        const uint32_t A = (uint32_t)(std::max_element(load.begin(), load.end()) - load.begin());
        const float LA = load[A];
        float best = LA - 1e-3f;
        int best_a = -1, best_b = -1;
        uint32_t best_B = 0;
        for (uint32_t ia = 0; ia < on[A].size(); ++ia) {
            const float a = size[on[A][ia]];
            for (uint32_t B = 0; B < m; ++B) {
                if (B == A) continue;
                const float moved = std::max(LA - a, load[B] + a);
                if (moved < best) {
                    best = moved;
                    best_a = (int)ia, best_b = -1, best_B = B;
                }
                for (uint32_t ib = 0; ib < on[B].size(); ++ib) {
                    const float b = size[on[B][ib]];
                    if (b >= a) continue;
                    const float swapped = std::max(LA - a + b, load[B] + a - b);
                    if (swapped < best) {
                        best = swapped;
                        best_a = (int)ia, best_b = (int)ib, best_B = B;
                    }
                }
            }
        }
        if (best_a < 0) break;
        const uint32_t qa = on[A][best_a];
        if (best_b >= 0) {
            const uint32_t qb = on[best_B][best_b];
            on[A][best_a] = qb;
            on[best_B][best_b] = qa;
            load[A] += size[qb] - size[qa];
            load[best_B] += size[qa] - size[qb];
        } else {
            on[A].erase(on[A].begin() + best_a);
            on[best_B].push_back(qa);
            load[A] -= size[qa];
            load[best_B] += size[qa];
        }
    }
    struct Job {
        float start;
        uint32_t q_tile;
    };
    std::vector<Job> jobs;
    jobs.reserve(n);
    for (uint32_t s = 0; s < m; ++s) {
        std::sort(on[s].begin(), on[s].end(), [&](uint32_t a, uint32_t b) { return size[a] > size[b]; });
        float t = 0.f;
        for (uint32_t q : on[s]) {
            jobs.push_back(Job{t, q});
            t += size[q];
        }
    }
    std::stable_sort(jobs.begin(), jobs.end(), [&](const Job &a, const Job &b) {
        return a.start != b.start ? a.start < b.start : size[a.q_tile] > size[b.q_tile];
    });
    std::vector<uint32_t> next_head(nq, 0);
    for (uint32_t i = 0; i < n; ++i) order[i] = (uint16_t)((jobs[i].q_tile << 8) | next_head[jobs[i].q_tile]++);
}

}  // namespace

// Returns MF_ERR_OPERATION_NOT_SUPPORTED (without touching last_error semantics) when the
// shape is outside this kernel's envelope; the caller then uses the mma.sync kernel.
mf_status launch_prefill_tc(MfContext *ctx, const void *q, const void *k, const void *v, void *out,
                            const SdpaPrefillSplitKParams &sp, bool *handled, const MfPagedKv *paged, uint32_t seq)
{
    *handled = false;
    const SdpaPrefillParams &b = sp.base;
    const uint32_t kD = b.head_dim;
    if ((kD != 64 && kD != 128) || std::max(1u, sp.split_k) != 1 || b.q_len < 64) return MF_OK;
    if (b.stride_k_s != kD || b.stride_v_s != kD) return MF_OK;
    if ((b.q_stride_m % 8) || (b.q_stride_h % 8) || (b.out_stride_m % 8) || (b.out_stride_h % 8)) return MF_OK;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out)) & 15u) return MF_OK;
    if (paged) {
        // pages of 8 to 128 rows (a power of two): a tile is a whole number of pages
        if (paged->page_size < 8 || paged->page_size > kBN) return MF_OK;
        k = paged->k_pool, v = paged->v_pool;
        if ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15u) return MF_OK;
    } else if (b.k_stride_h % 8 || b.v_stride_h % 8 ||
               (reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15u) {
        return MF_OK;
    }
    if (!ctx->encode_fn) {
        cudaDriverEntryPointQueryResult qr;
        void *fn = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) != cudaSuccess ||
            qr != cudaDriverEntryPointSuccess || !fn)
            return fail(ctx, MF_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
        ctx->encode_fn = fn;
    }
    typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    // (64 columns, rows, 2 column halves, heads) views with the caller's row and head strides: one box of
    // 64 columns x 128 rows x 2 halves brings a whole tile and lands as [half][row][128 B].
    auto encode = [&](CUtensorMap *tm, const void *base, uint64_t rows, uint64_t heads, uint64_t row_stride,
                      uint64_t head_stride, uint32_t box_rows = 128) {
        cuuint64_t gdim[4] = {64, rows, kD / 64, heads};
        cuuint64_t gstride[3] = {row_stride * 2, 128, head_stride * 2};
        cuuint32_t box[4] = {64, box_rows, kD / 64, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        return reinterpret_cast<EncodeFn>(ctx->encode_fn)(
                   tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void *>(base), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    };
    const uint32_t cache_heads = sp.n_heads / b.group_size;
    CUtensorMap tm_q, tm_k, tm_v;
    mf_status st;
    // Unusual strides the encoder refuses are left to the other kernel.
    if (!encode(&tm_q, q, b.q_len, sp.n_heads, b.q_stride_m, b.q_stride_h)) return MF_OK;
    if (paged) {
        // pool [n_pages, Hkv, P, D] as (64 columns, P rows, column halves, page x kv head); one copy = one
        // column half of one page of one kv head
        auto encode_pool = [&](CUtensorMap *tm, const void *base, uint32_t halves_per_copy) {
            const uint64_t P = paged->page_size;
            cuuint64_t gdim[4] = {64, P, kD / 64, (uint64_t)paged->n_pages * paged->n_kv_heads};
            cuuint64_t gstride[3] = {(uint64_t)kD * 2, 128, P * kD * 2};
            cuuint32_t box[4] = {64, (cuuint32_t)P, halves_per_copy, 1};
            cuuint32_t estr[4] = {1, 1, 1, 1};
            return reinterpret_cast<EncodeFn>(ctx->encode_fn)(
                       tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void *>(base), gdim, gstride, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
        };
        // K by column half (its descriptor needs the 128 rows of a half evenly spaced), V by whole page
        if (!encode_pool(&tm_k, k, 1) || !encode_pool(&tm_v, v, kD / 64)) return MF_OK;
    } else {
        if (!encode(&tm_k, k, b.kv_len, cache_heads, kD, b.k_stride_h, 128)) return MF_OK;
        if (!encode(&tm_v, v, b.kv_len, cache_heads, kD, b.v_stride_h, 128)) return MF_OK;
    }
    TcParams p{};
    if (paged) {
        p.page_table_row = paged->page_table + (size_t)seq * paged->page_table_stride;
        p.page_size = paged->page_size;
        for (p.page_shift = 0; (1u << p.page_shift) < paged->page_size; ++p.page_shift) {}
        p.n_kv_heads = paged->n_kv_heads;
    }
    p.out = static_cast<__half *>(out);
    p.status = ctx->d_status;
    p.q_len = b.q_len;
    p.kv_len = b.kv_len;
    p.query_offset = b.query_offset;
    p.group = b.group_size;
    p.out_stride_h = b.out_stride_h;
    p.out_stride_m = b.out_stride_m;
    p.scale_log2 = b.scale * 1.4426950408889634f;
    static bool configured[64][4] = {};
    const int di = (kD == 128 ? 1 : 0) + (paged ? 2 : 0);
    const uint32_t smem_bytes = tc_smem_bytes(kD);
    void (*kern)(CUtensorMap, CUtensorMap, CUtensorMap, TcParams) =
        di == 0 ? prefill_tc_kernel<64, false> : di == 1 ? prefill_tc_kernel<128, false>
        : di == 2 ? prefill_tc_kernel<64, true> : prefill_tc_kernel<128, true>;
    if (ctx->device < 64 && !configured[ctx->device][di]) {
        st = check_cuda(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes),
                        "cudaFuncSetAttribute(prefill_tc)");
        if (st != MF_OK) return st;
        configured[ctx->device][di] = true;
    }
    p.n_heads = sp.n_heads;
    p.n_q_tiles = (b.q_len + kBM - 1) / kBM;
    const uint32_t n_items = p.n_q_tiles * sp.n_heads;
    if (n_items <= 512 && p.n_q_tiles <= 256 && sp.n_heads <= 256 && n_items > (uint32_t)std::max(1, ctx->sm_count)) {
        // the list of the last shape is kept: the layers of a model launch the same shape one after another
        const uint32_t key[6] = {p.q_len, p.kv_len, p.query_offset, sp.n_heads, (uint32_t)ctx->sm_count, 1u};
        if (memcmp(key, ctx->tc_order_key, sizeof(key)) != 0 || ctx->tc_order_n != n_items) {
            tc_item_order(p, (uint32_t)ctx->sm_count, ctx->tc_order);
            memcpy(ctx->tc_order_key, key, sizeof(key));
            ctx->tc_order_n = n_items;
        }
        memcpy(p.order, ctx->tc_order, n_items * sizeof(uint16_t));
        p.use_order = 1;
    }
    dim3 grid(n_items);
    kern<<<grid, kTcThreads, smem_bytes, ctx->stream>>>(tm_q, tm_k, tm_v, p);
    *handled = true;
    return check_launch(ctx, "prefill_tc_kernel");
}

}  // namespace mf
