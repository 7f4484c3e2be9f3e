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
#include "append.cuh"
#include "internal.hpp"
#include "ptx.cuh"

namespace mf {
namespace {

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
    rope_and_store(p, s, slot, j, a, c);
}

// RMSNorm -> Q/K/V projection (+bias) with f16 weights, optionally followed by the append above
// (qkv_project.metal:4-272 computes the projection with one warp per output row and scalar FMAs).
// Here a CTA owns one chunk pair of one head slot: the 16 output rows [8j, 8j+8) and
// [8j + D/2, 8j + D/2 + 8) of a head, which is exactly what one thread of kv_append_kernel consumes,
// for up to eight input rows, and the products run on mma.sync m16n8k16 (f16 in, f32 accumulate):
// the 16 weight rows are the m side, the input rows the n side.  Warp w takes the 32-wide k blocks
// w, w+8, ...; lane l reads 16 bytes of row l/4 of each row group at k quarter l%4 (in the blocked
// weight layout the eight rows of a group are 512 contiguous bytes per k block: one full line per
// warp load) and uses them directly as its A fragments of two mma steps; the k order inside a step
// is therefore permuted, the same way for the input fragment read from shared memory, which leaves
// the dot product unchanged.  A row's sum = the warp's accumulator chain over its k blocks, then the
// eight warps added in order: independent of the number of input rows and of the append.
constexpr uint32_t kQkvRows = 8;   // the n side of the mma
constexpr int kQkvDepth = 4;       // k blocks per register buffer; two buffers in flight
constexpr uint32_t kQkvPad = 32;   // halves between staged rows beyond K: rows 64 bytes apart modulo 128

struct QkvWeights {
    uint4 lo[kQkvDepth], hi[kQkvDepth];
};

__device__ __forceinline__ void cp_async_16(void *smem_dst, const void *gmem_src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)),
                 "l"(gmem_src)
                 : "memory");
}
__device__ __forceinline__ void cp_async_wait_all()
{
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}


// What a CTA needs to know about one slab (chunk pair j of head slot `slot`).
struct QkvSlab {
    const __half *wl_lo, *wl_hi, *bias;  // this lane's weight pointers (k block 0), bias of the matrix
    __half *plain;                       // optional projected output of the matrix
    size_t kb_stride;
    uint32_t n, slot, j, first_row;      // first_row: of row group 0; group 1 is head_dim/2 further
};

__global__ void __launch_bounds__(256, 2) fused_qkv_kernel(const QkvParams qp, const AppendParams ap)
{
    extern __shared__ __align__(16) unsigned char qkv_smem[];
    __half *xs = reinterpret_cast<__half *>(qkv_smem);  // [rows_per_cta][K + pad], normalised
    __shared__ float red[8][16][kQkvRows];
    __shared__ float ssq[8][kQkvRows];
    __shared__ __align__(16) __half outv[kQkvRows][16];

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t cpr = qp.head_dim / 16;
    const uint32_t n_slabs = (qp.q_slots + 2 * qp.kv_slots) * cpr;
    const uint32_t row0 = blockIdx.y * qp.rows_per_cta;
    const uint32_t rows = min(qp.rows_per_cta, qp.m - row0);
    const uint32_t K = qp.k_dim, xstride = K + kQkvPad, nkb = K / 32;
    const uint32_t r_in = lane >> 2, kq = lane & 3;

    auto describe = [&](uint32_t slab) {
        QkvSlab d;
        d.slot = slab / cpr, d.j = slab % cpr;
        const __half *w;
        uint32_t head;
        if (d.slot < qp.q_slots) {
            w = qp.w_q, d.bias = qp.b_q, d.plain = qp.out_q, d.n = qp.n_dim, head = d.slot;
        } else if (d.slot < qp.q_slots + qp.kv_slots) {
            w = qp.w_k, d.bias = qp.b_k, d.plain = qp.out_k, d.n = qp.n_kv, head = d.slot - qp.q_slots;
        } else {
            w = qp.w_v, d.bias = qp.b_v, d.plain = qp.out_v, d.n = qp.n_kv, head = d.slot - qp.q_slots - qp.kv_slots;
        }
        d.first_row = head * qp.head_dim + 8 * d.j;
        const uint32_t row_lo = d.first_row + r_in, row_hi = row_lo + qp.head_dim / 2;
        d.wl_lo = qp.blocked ? w + (size_t)row_lo * 32 + kq * 8 : w + (size_t)row_lo * K + kq * 8;
        d.wl_hi = qp.blocked ? w + (size_t)row_hi * 32 + kq * 8 : w + (size_t)row_hi * K + kq * 8;
        d.kb_stride = qp.blocked ? (size_t)d.n * 32 : 32;
        return d;
    };
    auto fetch = [&](QkvWeights &dst, const QkvSlab &d, uint32_t chunk) {
#pragma unroll
        for (int u = 0; u < kQkvDepth; ++u) {
            const uint32_t kb = warp + 8 * (chunk * kQkvDepth + u);
            if (kb < nkb) {
                dst.lo[u] = __ldg(reinterpret_cast<const uint4 *>(d.wl_lo + kb * d.kb_stride));
                dst.hi[u] = __ldg(reinterpret_cast<const uint4 *>(d.wl_hi + kb * d.kb_stride));
            } else {
                dst.lo[u] = dst.hi[u] = make_uint4(0, 0, 0, 0);
            }
        }
    };

    if (!qp.strict_release) grid_launch_dependents();
    // The weights are constants: the first 64 KB of them are requested before the grid waits for the
    // kernel in front of it (under a programmatic dependent launch they travel during its tail) and
    // keep arriving while the input rows are staged and normalised.
    uint32_t slab = blockIdx.x;
    QkvSlab sd = describe(slab);
    QkvWeights cur, nxt;
    fetch(cur, sd, 0);
    fetch(nxt, sd, 1);
    grid_dependency_wait();  // from here on: reads of what that kernel may have produced, and writes
    // a strict launch releases the next one only now (the bound the decode kernel's early K/V stream relies on)
    if (qp.strict_release) grid_launch_dependents();
    const uint32_t vecs = K / 8;
    __half *gs = xs + (size_t)qp.rows_per_cta * xstride;  // gamma, staged once
    for (uint32_t b = 0; b < rows; ++b)
        for (uint32_t i = tid; i < vecs; i += 256)
            cp_async_16(xs + (size_t)b * xstride + 8 * i, qp.x + (size_t)(row0 + b) * K + 8 * i);
    if (qp.gamma)
        for (uint32_t i = tid; i < vecs; i += 256) cp_async_16(gs + 8 * i, qp.gamma + 8 * i);
    cp_async_wait_all();
    if (qp.gamma) {
        // each thread squares, and later scales, the vectors it copied itself
        for (uint32_t b = 0; b < rows; ++b) {
            float sq = 0.f;
            for (uint32_t i = tid; i < vecs; i += 256) {
                Chunk c;
                c.u = *reinterpret_cast<const uint4 *>(xs + (size_t)b * xstride + 8 * i);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float f = __half2float(c.h[e]);
                    sq = fmaf(f, f, sq);
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (lane == 0) ssq[warp][b] = sq;
        }
        __syncthreads();
        for (uint32_t b = 0; b < rows; ++b) {
            float t = 0.f;
#pragma unroll
            for (int wv = 0; wv < 8; ++wv) t += ssq[wv][b];
            const float inv = 1.0f / sqrtf(t / (float)K + qp.eps);
            for (uint32_t i = tid; i < vecs; i += 256) {
                Chunk c, g;
                c.u = *reinterpret_cast<const uint4 *>(xs + (size_t)b * xstride + 8 * i);
                g.u = *reinterpret_cast<const uint4 *>(gs + 8 * i);
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    c.h[e] = __float2half_rn(__fmul_rn(__fmul_rn(__half2float(c.h[e]), inv), __half2float(g.h[e])));
                *reinterpret_cast<uint4 *>(xs + (size_t)b * xstride + 8 * i) = c.u;
            }
        }
    }
    __syncthreads();

    const bool has_x = r_in < rows;  // this lane's input row on the n side
    const __half *xl = xs + (size_t)r_in * xstride + kq * 8;
    const uint32_t per_warp = (nkb + 7 - warp) / 8;
    const uint32_t chunks = (per_warp + kQkvDepth - 1) / kQkvDepth;
    for (;;) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (uint32_t chunk = 0; chunk < chunks; ++chunk) {
#pragma unroll
            for (int u = 0; u < kQkvDepth; ++u) {
                const uint32_t kb = warp + 8 * (chunk * kQkvDepth + u);
                if (kb < nkb) {
                    const uint4 xv = has_x ? *reinterpret_cast<const uint4 *>(xl + kb * 32) : make_uint4(0, 0, 0, 0);
                    const uint32_t a1[4] = {cur.lo[u].x, cur.hi[u].x, cur.lo[u].y, cur.hi[u].y};
                    mma_m16n8k16(acc, a1, xv.x, xv.y);
                    const uint32_t a2[4] = {cur.lo[u].z, cur.hi[u].z, cur.lo[u].w, cur.hi[u].w};
                    mma_m16n8k16(acc, a2, xv.z, xv.w);
                }
            }
            cur = nxt;
            if (chunk + 2 < chunks) fetch(nxt, sd, chunk + 2);
        }
        red[warp][r_in][2 * kq] = acc[0];
        red[warp][r_in][2 * kq + 1] = acc[1];
        red[warp][r_in + 8][2 * kq] = acc[2];
        red[warp][r_in + 8][2 * kq + 1] = acc[3];
        // the next slab's weights travel during this slab's reduction and stores
        const QkvSlab done = sd;
        slab += gridDim.x;
        const bool more = slab < n_slabs;
        if (more) {
            sd = describe(slab);
            fetch(cur, sd, 0);
            fetch(nxt, sd, 1);
        }
        __syncthreads();
        if (tid < 16 * kQkvRows) {
            const uint32_t r = tid & 15, b = tid >> 4;
            float sum = red[0][r][b];
#pragma unroll
            for (int wv = 1; wv < 8; ++wv) sum += red[wv][r][b];
            if (done.bias) sum += __half2float(done.bias[done.first_row + (r >> 3) * (qp.head_dim / 2) + (r & 7)]);
            outv[b][r] = __float2half_rn(sum);
        }
        __syncthreads();
        if (tid < rows) {
            const uint32_t s = row0 + tid;
            Chunk a, c;
            a.u = *reinterpret_cast<const uint4 *>(&outv[tid][0]);
            c.u = *reinterpret_cast<const uint4 *>(&outv[tid][8]);
            if (done.plain) {
                __half *dst = done.plain + (size_t)s * done.n + done.first_row;
                *reinterpret_cast<uint4 *>(dst) = a.u;
                *reinterpret_cast<uint4 *>(dst + qp.head_dim / 2) = c.u;
            }
            if (qp.append) rope_and_store(ap, s, done.slot, done.j, a, c);
        }
        if (!more) break;
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
                  uint32_t max_seq_len, const uint32_t *page_table_row, uint32_t page_size, uint32_t out_rows,
                  uint32_t n_pages = 0, uint32_t *status = nullptr)
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
        if (page >= n_pages) {  // not a page of this pool: the row reads as zero, the status word says why
            atomicOr(status, kStatusBadPage);
            *reinterpret_cast<uint4 *>(out + ((size_t)h * out_rows + t) * head_dim + 8 * j) = make_uint4(0, 0, 0, 0);
            return;
        }
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
                      uint32_t max_seq_len, const uint32_t *page_table_row, uint32_t page_size, uint32_t n_pages,
                      uint32_t *status)
{
    const uint32_t cpr = head_dim / 8;
    const uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (uint64_t)heads * len * cpr) return;
    const uint32_t j = gid % cpr;
    const uint32_t t = (gid / cpr) % len;
    const uint32_t h = gid / ((uint64_t)cpr * len);
    const uint32_t page = page_table_row[t / page_size];
    if (page >= n_pages) {
        atomicOr(status, kStatusBadPage);
        return;
    }
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
                  uint32_t n, uint64_t chunks_per_page, uint32_t n_pages, uint32_t *status)
{
    const uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (uint64_t)n * chunks_per_page * 2) return;
    const uint64_t c = gid % chunks_per_page;
    const uint64_t pi = gid / chunks_per_page;
    uint4 *pool = (pi & 1) ? v_pool : k_pool;
    const uint32_t i = (uint32_t)(pi >> 1);
    const uint32_t src = src_ids[i], dst = dst_ids[i];
    if (src >= n_pages || dst >= n_pages) {
        atomicOr(status, kStatusBadPage);
        return;
    }
    pool[(uint64_t)dst * chunks_per_page + c] = pool[(uint64_t)src * chunks_per_page + c];
}

inline uint32_t blocks_for(uint64_t threads) { return (uint32_t)((threads + 255) / 256); }

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace mf

using namespace mf;

extern "C" {

// Checks and kernel parameters of KvPrepFused.  with_inputs == false: q, k, v come from a
// projection inside the launch and are not looked at.
static mf_status kv_prep_params(MfContext *ctx, const MfTensor *q, const MfTensor *k, const MfTensor *v,
                                const MfTensor *q_rot, const MfTensor *k_cache, const MfTensor *v_cache,
                                const MfTensor *cos, const MfTensor *sin, const KvPrepFusedParamsResolved *pr,
                                bool with_inputs, AppendParams &p)
{
    if (!pr) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "params");
    mf_status st;
    const MfTensor *ts[8] = {q, k, v, q_rot, k_cache, v_cache, cos, sin};
    const char *names[8] = {"q", "k", "v", "q_rot", "k_cache", "v_cache", "cos", "sin"};
    for (int i = with_inputs ? 0 : 3; i < 8; ++i)
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
    p = AppendParams{};
    p.q = with_inputs ? tensor_ptr(q) : nullptr;
    p.k = with_inputs ? tensor_ptr(k) : nullptr;
    p.v = with_inputs ? tensor_ptr(v) : nullptr;
    p.q_rot = tensor_ptr(q_rot);
    p.k_cache = tensor_ptr(k_cache);
    p.v_cache = tensor_ptr(v_cache);
    p.cos_t = tensor_ptr(cos);
    p.sin_t = tensor_ptr(sin);
    const void *ptrs[8] = {p.q, p.k, p.v, p.q_rot, p.k_cache, p.v_cache, p.cos_t, p.sin_t};
    for (int i = with_inputs ? 0 : 3; i < 8; ++i)
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
    return MF_OK;
}

mf_status mf_kv_prep_fused(MfContext *ctx, const MfTensor *q, const MfTensor *k, const MfTensor *v,
                           const MfTensor *q_rot, const MfTensor *k_cache, const MfTensor *v_cache,
                           const MfTensor *cos, const MfTensor *sin, const KvPrepFusedParamsResolved *pr)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    AppendParams p;
    const mf_status st = kv_prep_params(ctx, q, k, v, q_rot, k_cache, v_cache, cos, sin, pr, true, p);
    if (st != MF_OK || p.seq_len == 0) return st;
    const uint64_t threads = (uint64_t)p.seq_len * (p.n_heads + 2 * p.n_kv_heads) * (p.head_dim / 16);
    kv_append_kernel<<<blocks_for(threads), 256, 0, ctx->stream>>>(p);
    return check_launch(ctx, "kv_append_kernel");
}

static mf_status paged_append_params(MfContext *ctx, const MfPagedKv *cache, const void *q, const void *k,
                                     const void *v, void *q_rot, const void *cos, const void *sin, uint32_t n_heads,
                                     uint32_t rope_mode, uint32_t apply_rope, uint32_t seq, uint32_t position_offset,
                                     uint32_t seq_len, bool with_inputs, AppendParams &p)
{
    if (!cache || !cache->k_pool || !cache->v_pool || !cache->page_table || (with_inputs && (!q || !k || !v)))
        return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged append: null input");
    if (apply_rope && (!cos || !sin)) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "paged append: cos/sin");
    if (cache->head_dim % 16 != 0 || cache->n_kv_heads == 0 || n_heads % cache->n_kv_heads != 0)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "paged append: geometry");
    if (rope_mode > 1) return fail(ctx, MF_ERR_INVALID_OPERATION, "paged append: rope_mode %u", rope_mode);
    p = AppendParams{};
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
    p.n_pages = cache->n_pages;
    p.status = ctx->d_status;
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
    return MF_OK;
}

mf_status mf_paged_kv_append(MfContext *ctx, const MfPagedKv *cache, const void *q, const void *k, const void *v,
                             void *q_rot, const void *cos, const void *sin, uint32_t n_heads, uint32_t rope_mode,
                             uint32_t apply_rope, uint32_t seq, uint32_t position_offset, uint32_t seq_len)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    AppendParams p;
    const mf_status st = paged_append_params(ctx, cache, q, k, v, q_rot, cos, sin, n_heads, rope_mode, apply_rope, seq,
                                             position_offset, seq_len, true, p);
    if (st != MF_OK || p.seq_len == 0) return st;
    const uint64_t threads = (uint64_t)p.seq_len * (p.n_heads + 2 * p.n_kv_heads) * (p.head_dim / 16);
    kv_append_kernel<<<blocks_for(threads), 256, 0, ctx->stream>>>(p);
    return check_launch(ctx, "kv_append_kernel(paged)");
}

// ---- FusedQkv and its two append forms -----------------------------------------------------------

static mf_status launch_fused_qkv(MfContext *ctx, const MfFusedQkvArgs *a, uint32_t head_dim, uint32_t q_slots,
                                  uint32_t kv_slots, const AppendParams *ap, bool want_plain, const char *what)
{
    if (!a->input || !a->w_q || !a->w_k || !a->w_v) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "%s: input / weights", what);
    if (want_plain && (!a->out_q || !a->out_k || !a->out_v)) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "%s: outputs", what);
    const bool any_bias = a->bias_q || a->bias_k || a->bias_v;
    if (any_bias && !(a->bias_q && a->bias_k && a->bias_v))
        return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "%s: give all three biases or none", what);
    if (a->weights_per_block != 0 && a->weights_per_block != 32)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "%s: weights_per_block %u (0 = row-major, 32 = blocked)", what,
                    a->weights_per_block);
    if (a->k_dim == 0 || a->k_dim % 32 != 0 || a->n_dim % 16 != 0 || a->n_kv % 16 != 0 || a->n_dim == 0)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "%s: k_dim %u must be a multiple of 32, n_dim %u and n_kv %u of 16", what,
                    a->k_dim, a->n_dim, a->n_kv);
    const void *ptrs[] = {a->input, a->w_q, a->w_k, a->w_v, a->gamma, a->bias_q, a->bias_k, a->bias_v,
                          a->out_q, a->out_k, a->out_v};
    for (const void *ptr : ptrs)
        if (ptr && !aligned16(ptr)) return fail(ctx, MF_ERR_INVALID_SHAPE, "%s: pointers must be 16-byte aligned", what);
    if (a->m == 0) return MF_OK;
    QkvParams qp{};
    qp.x = static_cast<const __half *>(a->input);
    qp.w_q = static_cast<const __half *>(a->w_q);
    qp.w_k = static_cast<const __half *>(a->w_k);
    qp.w_v = static_cast<const __half *>(a->w_v);
    qp.gamma = static_cast<const __half *>(a->gamma);
    qp.b_q = static_cast<const __half *>(a->bias_q);
    qp.b_k = static_cast<const __half *>(a->bias_k);
    qp.b_v = static_cast<const __half *>(a->bias_v);
    qp.out_q = static_cast<__half *>(a->out_q);
    qp.out_k = static_cast<__half *>(a->out_k);
    qp.out_v = static_cast<__half *>(a->out_v);
    qp.k_dim = a->k_dim, qp.n_dim = a->n_dim, qp.n_kv = a->n_kv, qp.m = a->m;
    qp.blocked = a->weights_per_block == 32;
    qp.head_dim = head_dim, qp.q_slots = q_slots, qp.kv_slots = kv_slots;
    qp.eps = a->epsilon;
    qp.append = ap != nullptr;
    const AppendParams none{};
    const AppendParams &app = ap ? *ap : none;
    // eight input rows or more: the tensor-core kernel (fused_qkv_tc.cu), when the shape is one it takes
    if (fused_qkv_tc_eligible(ctx, qp)) return launch_fused_qkv_tc(ctx, qp, app, what);
    // input rows per CTA: eight, fewer when the staged rows would not fit in shared memory
    const size_t row_bytes = ((size_t)a->k_dim + kQkvPad) * sizeof(__half), budget = 200 * 1024;
    if (2 * row_bytes > budget) return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "%s: k_dim %u too large", what, a->k_dim);
    uint32_t rows = a->m < kQkvRows ? a->m : kQkvRows;
    while ((rows + 1) * row_bytes > budget) --rows;  // + 1: gamma
    qp.rows_per_cta = rows;
    // CTAs loop over slabs; two CTAs are resident per SM
    const uint32_t slabs = (q_slots + 2 * kv_slots) * (head_dim / 16), tiles = (a->m + rows - 1) / rows;
    const size_t smem = rows * row_bytes + (a->gamma ? (size_t)a->k_dim * sizeof(__half) : 0);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(fused_qkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget) != cudaSuccess)
        return fail(ctx, MF_ERR_OPERATION_NOT_SUPPORTED, "%s: cannot get %zu bytes of shared memory", what, smem);
    const uint32_t resident = std::max(1u, 2u * (uint32_t)ctx->sm_count / tiles);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(std::min(slabs, resident), tiles, 1);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    cfg.attrs = attr;
    cfg.numAttrs = 0;
    if (ctx->overlap_launches) {
        // programmatic dependent launch: the grid may be scheduled while the kernel before it drains;
        // it waits before it reads or writes anything
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 1;
        qp.strict_release = ctx->next_launch_strict() ? 1u : 0u;
    }
    const cudaError_t e = cudaLaunchKernelEx(&cfg, fused_qkv_kernel, qp, app);
    if (e != cudaSuccess) return fail(ctx, MF_ERR_CUDA, "launch fused_qkv_kernel: %s", cudaGetErrorString(e));
    ++ctx->launches;
    // this kernel releases its dependents before it ends: a decode launch behind it must not stream the
    // caches it is writing ahead of its own dependency wait
    if (ctx->overlap_launches)
        ctx->note_programmatic_launch(qp.strict_release != 0, ap ? ap->k_cache : nullptr, ap ? ap->v_cache : nullptr);
    return MF_OK;
}

mf_status mf_fused_qkv(MfContext *ctx, const MfFusedQkvArgs *args)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!args) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "FusedQkv: args");
    return launch_fused_qkv(ctx, args, 16, args->n_dim / 16, args->n_kv / 16, nullptr, true, "FusedQkv");
}

mf_status mf_fused_qkv_kv_prep(MfContext *ctx, const MfFusedQkvArgs *args, const MfTensor *q_rot,
                               const MfTensor *k_cache, const MfTensor *v_cache, const MfTensor *cos,
                               const MfTensor *sin, const KvPrepFusedParamsResolved *pr)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!args) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "FusedQkv+KvPrepFused: args");
    AppendParams p;
    const mf_status st = kv_prep_params(ctx, nullptr, nullptr, nullptr, q_rot, k_cache, v_cache, cos, sin, pr, false, p);
    if (st != MF_OK) return st;
    if (args->m != pr->seq_len || args->n_dim != pr->d_model || args->n_kv != pr->kv_dim)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "FusedQkv+KvPrepFused: m %u / n_dim %u / n_kv %u against seq_len %u / d_model %u / kv_dim %u",
                    args->m, args->n_dim, args->n_kv, pr->seq_len, pr->d_model, pr->kv_dim);
    return launch_fused_qkv(ctx, args, p.head_dim, p.n_heads, p.n_kv_heads, &p, false, "FusedQkv+KvPrepFused");
}

mf_status mf_fused_qkv_paged_append(MfContext *ctx, const MfFusedQkvArgs *args, const MfPagedKv *cache, void *q_rot,
                                    const void *cos, const void *sin, uint32_t n_heads, uint32_t rope_mode,
                                    uint32_t apply_rope, uint32_t seq, uint32_t position_offset)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!args) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "FusedQkv+paged append: args");
    AppendParams p;
    const mf_status st = paged_append_params(ctx, cache, nullptr, nullptr, nullptr, q_rot, cos, sin, n_heads, rope_mode,
                                             apply_rope, seq, position_offset, args->m, false, p);
    if (st != MF_OK) return st;
    if (args->m != p.seq_len || args->n_dim != n_heads * p.head_dim || args->n_kv != p.n_kv_heads * p.head_dim)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "FusedQkv+paged append: m %u / n_dim %u / n_kv %u against the cache geometry",
                    args->m, args->n_dim, args->n_kv);
    return launch_fused_qkv(ctx, args, p.head_dim, p.n_heads, p.n_kv_heads, &p, false, "FusedQkv+paged append");
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
        paged->page_table + (size_t)seq * paged->page_table_stride, paged->page_size, paged->n_pages, ctx->d_status);
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
        static_cast<uint4 *>(cache->k_pool), static_cast<uint4 *>(cache->v_pool), src_ids, dst_ids, n, chunks,
        cache->n_pages, ctx->d_status);
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
        cache->page_table + (size_t)seq * cache->page_table_stride, cache->page_size, len, cache->n_pages, ctx->d_status);
    return check_launch(ctx, "cache_read_kernel(paged)");
}

}  // extern "C"
