// Sequence-sharded decode: what a decode kernel's consumer threads do to hand a finished unit's partial
// (acc, m, l) to every rank and, in the fused form, to merge all ranks' partials themselves.  Shared by
// the f16 and the 8-bit decode kernels; both run these with 128 consumer threads and the named barriers
// 1 and 2 of their CTA.
#pragma once

#include "internal.hpp"
#include "ptx.cuh"

namespace mf {
namespace push {

constexpr uint32_t kConsumerThreads = 128;
constexpr float kNegSentinel = -1e30f;

// One value of a partial into rank r's receive block.  Tagged form: value and step tag in ONE 64-bit store, which
// the reader sees whole or not at all; it trusts the word once it carries this step's tag, so neither a fence nor a
// counter stands between the stores and the merge (a system-scope fence costs about 5 us on this machine).
__device__ __forceinline__ void push_store(const DecodeParams &p, uint32_t r, size_t e, float v)
{
    if (p.push_tagged) {
        // one scalar 64-bit store (tag in the low word): single-copy atomic by the memory model, not only in practice
        const unsigned long long word = ((unsigned long long)__float_as_uint(v) << 32) | p.push_tag;
        asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(reinterpret_cast<unsigned long long *>(p.push_dst[r]) + e), "l"(word) : "memory");
    } else {
        p.push_dst[r][e] = v;
    }
}
// A tagged word of this rank's receive blocks; false while it does not carry the tag yet.
__device__ __forceinline__ bool tagged_load(const float *base, size_t e, uint32_t tag, float &v)
{
    unsigned long long word;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(word) : "l"(reinterpret_cast<const unsigned long long *>(base) + e) : "memory");
    v = __uint_as_float((uint32_t)(word >> 32));
    return (uint32_t)word == tag;
}

// Sequence-sharded decode, end of a unit: announce the block this CTA has just stored into every
// rank's receive buffer; with push_merge also wait (bounded) until every pushing rank has delivered
// the same unit, merge the unit's query heads out of local memory (flash_prefill.metal:843-888)
// and write the output rows.  Called by all consumer threads.
// Sequence-sharded decode, before a CTA's first push of a launch: ranks that only merge never wait for
// anybody, so this is what keeps a pusher from overwriting the parity block such a rank still reads.
// Polls this rank's own memory (the merging rank counts its merged rows there), bounded.
__device__ __forceinline__ void push_wait_for_mergers(const DecodeParams &p, uint32_t tid)
{
    if (tid == 0) {
        const long long t0 = clock64();
        for (uint32_t r = 0; r < 8; ++r) {
            if (!(p.push_wait_mask >> r & 1u)) continue;
            uint32_t spins = 0;
            for (;;) {
                uint32_t v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.push_merged_local + r) : "memory");
                if ((int32_t)(v - p.push_wait_expected) >= 0) break;
                if ((++spins & 0x3Fu) == 0 && clock64() - t0 > 4000000000ll) {
                    atomicOr(p.status, kStatusPushWait);
                    break;
                }
            }
        }
    }
    named_bar_sync(2, kConsumerThreads);
}

template <int D>
__device__ __forceinline__ void push_signal_and_merge(const DecodeParams &p, const WorkItem &it, uint32_t tid,
                                                      volatile uint32_t *flags)
{
    if (p.push_tagged) {
        // Tagged words: every value of every pushing rank's block is read until it carries this step's tag (all loads
        // of a column in flight together, bounded), then merged.  Nothing else to wait for.  The arrival counters
        // still advance (unfenced: nobody reads them in this form), so that a later step in the counted form
        // finds the totals it expects.
        if (tid < p.push_world) {
            atomicAdd_system(p.push_cnt[tid], 1u);
            atomicAdd_system(p.push_unit_cnt[tid] + it.unit, 1u);
        }
        const uint32_t G = p.group;
        const size_t rows = (size_t)p.batch * p.n_heads;
        const size_t block = rows * (D + 2);
        const uint32_t cols4 = G * (D / 4);
        for (uint32_t c4 = tid; c4 < cols4; c4 += kConsumerThreads) {
            const uint32_t g2 = c4 / (D / 4), d0 = (c4 % (D / 4)) * 4;
            const uint32_t h = it.kvh * G + g2;
            const size_t rowi = (size_t)it.seq * p.n_heads + h;
            float mr[8], lr[8], av[8][4];
            const long long t0 = clock64();
            bool all;
            uint32_t spins = 0;
            do {
                all = true;
#pragma unroll
                for (uint32_t r = 0; r < 8; ++r) {
                    if (r < p.push_world && (p.push_mask >> r & 1u)) {
                        all &= tagged_load(p.push_local, r * block + rows * D + rowi, p.push_tag, mr[r]);
                        all &= tagged_load(p.push_local, r * block + rows * D + rows + rowi, p.push_tag, lr[r]);
#pragma unroll
                        for (uint32_t i = 0; i < 4; ++i) all &= tagged_load(p.push_local, r * block + rowi * D + d0 + i, p.push_tag, av[r][i]);
                    } else {
                        mr[r] = kNegSentinel;
                        lr[r] = av[r][0] = av[r][1] = av[r][2] = av[r][3] = 0.f;
                    }
                }
            } while (!all && !((++spins & 0x3Fu) == 0 && clock64() - t0 > 4000000000ll));
            if (!all) atomicOr(p.status, 2048u);
            float mx = kNegSentinel;
#pragma unroll
            for (uint32_t r = 0; r < 8; ++r) mx = fmaxf(mx, mr[r]);
            float lt = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (uint32_t r = 0; r < 8; ++r) {
                if (r < p.push_world && (p.push_mask >> r & 1u)) {
                    const float w = __expf(mr[r] - mx);
                    if (lr[r] > 0.f) lt += lr[r] * w;
                    acc.x += av[r][0] * w;
                    acc.y += av[r][1] * w;
                    acc.z += av[r][2] * w;
                    acc.w += av[r][3] * w;
                }
            }
            const float inv = ((fabsf(lt) <= 3.0e38f) && fabsf(lt) > 1e-6f) ? 1.0f / lt : 0.f;
            __half *dst = p.out + (size_t)it.seq * p.out_stride_b + (size_t)h * p.out_stride_h + d0;
            dst[0] = __float2half_rn(acc.x * inv);
            dst[1] = __float2half_rn(acc.y * inv);
            dst[2] = __float2half_rn(acc.z * inv);
            dst[3] = __float2half_rn(acc.w * inv);
        }
        return;
    }
    // Every peer sees this unit's block before its counters move: the CTA's (and, in the cluster form, the
    // cluster's) stores happen before this barrier, the barrier before the signalling threads' system-scope fence,
    // and fences are cumulative.  Only those threads execute one: it costs microseconds, whatever is outstanding.
    named_bar_sync(1, kConsumerThreads);
    if (tid < p.push_world) {
        __threadfence_system();
        atomicAdd_system(p.push_cnt[tid], 1u);
        atomicAdd_system(p.push_unit_cnt[tid] + it.unit, 1u);
    }
    if (!p.push_merge) return;
    // push_local_cnt is this rank's own counter array: the wait polls local memory, never NVLink
    if (tid == 0) {
        uint32_t good = 1, spins = 0;
        const long long t0 = clock64();
        for (;;) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.push_local_cnt + it.unit) : "memory");
            if ((int32_t)(v - p.push_expected) >= 0) break;
            if ((++spins & 0x3Fu) == 0 && clock64() - t0 > 4000000000ll) {
                good = 0;
                atomicOr(p.status, 2048u);
                break;
            }
        }
        flags[1] = good;
    }
    named_bar_sync(2, kConsumerThreads);
    if (!flags[1]) return;
    const uint32_t G = p.group;
    const size_t rows = (size_t)p.batch * p.n_heads;
    const size_t block = rows * (D + 2);
    const uint32_t cols4 = G * (D / 4);
    for (uint32_t c4 = tid; c4 < cols4; c4 += kConsumerThreads) {
        const uint32_t g2 = c4 / (D / 4), d0 = (c4 % (D / 4)) * 4;
        const uint32_t h = it.kvh * G + g2;
        const size_t rowi = (size_t)it.seq * p.n_heads + h;
        float mr[8], lr[8];
        float mx = kNegSentinel;
#pragma unroll
        for (uint32_t r = 0; r < 8; ++r) {
            if (r < p.push_world && (p.push_mask >> r & 1u)) {
                mr[r] = __ldcg(p.push_local + r * block + rows * D + rowi);
                lr[r] = __ldcg(p.push_local + r * block + rows * D + rows + rowi);
                mx = fmaxf(mx, mr[r]);
            } else {
                mr[r] = kNegSentinel;
                lr[r] = 0.f;
            }
        }
        float lt = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (uint32_t r = 0; r < 8; ++r) {
            if (r < p.push_world && (p.push_mask >> r & 1u)) {
                const float w = __expf(mr[r] - mx);
                if (lr[r] > 0.f) lt += lr[r] * w;
                const float4 a = __ldcg(reinterpret_cast<const float4 *>(p.push_local + r * block + rowi * D + d0));
                acc.x += a.x * w;
                acc.y += a.y * w;
                acc.z += a.z * w;
                acc.w += a.w * w;
            }
        }
        const float inv = ((fabsf(lt) <= 3.0e38f) && fabsf(lt) > 1e-6f) ? 1.0f / lt : 0.f;
        __half *dst = p.out + (size_t)it.seq * p.out_stride_b + (size_t)h * p.out_stride_h + d0;
        dst[0] = __float2half_rn(acc.x * inv);
        dst[1] = __float2half_rn(acc.y * inv);
        dst[2] = __float2half_rn(acc.z * inv);
        dst[3] = __float2half_rn(acc.w * inv);
    }
}

}  // namespace push
}  // namespace mf
