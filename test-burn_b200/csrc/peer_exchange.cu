// Sequence-sharded decode without a library collective: buffers that every rank's decode
// kernel stores its partials into (over NVLink, through CUDA IPC mappings), and the merge
// kernel that waits for them.  No counterpart in the reference, whose engine is one GPU.
#include <cuda_fp16.h>
#include <dlfcn.h>

#include "internal.hpp"
#include "ptx.cuh"

namespace mf {
namespace {

// Counter region in front of the receive blocks: 8 per-source totals, 8 "merged by rank m" counts
// (the back-pressure of ranks that only merge), then one counter per unit (units <= rows), padded so
// that the floats stay 256-byte aligned.
inline size_t counter_bytes(uint32_t rows) { return ((size_t)(kPeerUnitCounters + rows) * 4 + 255) & ~(size_t)255; }

struct PushedMergeArgs {
    const float *gather;       // this rank's receive buffer, parity already applied: [world][block]
    const uint32_t *counters;  // this rank's arrival counters [world]
    uint32_t expected[8];      // counter value that completes the step, 0 = rank sends nothing
    uint32_t world, rows, head_dim;
    uint64_t block;            // floats per source rank
    uint32_t *status;
    // A rank that only merges tells the pushers when it is done with a step's blocks: one count per
    // merged row on every other rank's "merged by" word for this rank (null = this rank also pushes).
    uint32_t *merged_dst[8];
    uint32_t strict_release;  // 1: dependents are released after the dependency wait, not at the start
};

// Merge of pushed partials: wait (bounded) for every source rank, then the log-sum-exp merge
// of flash_prefill.metal:843-888 out of local memory.
__global__ void __launch_bounds__(128) merge_pushed_kernel(const PushedMergeArgs a, __half *__restrict__ out)
{
    __shared__ uint32_t ok;
    const uint32_t row = blockIdx.x;
    // Launched as a programmatic dependent of this rank's decode kernel, so it may be resident
    // while that kernel still runs (all of whose CTAs are resident by then, so it cannot be starved).
    // The arrival counters are the real dependency.
    if (!a.strict_release) grid_launch_dependents();
    if (threadIdx.x == 0) {
        uint32_t good = 1;
        const long long t0 = clock64();
        for (uint32_t r = 0; r < a.world && good; ++r) {
            if (!a.expected[r]) continue;
            uint32_t spins = 0;
            for (;;) {
                uint32_t v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a.counters + r) : "memory");
                if ((int32_t)(v - a.expected[r]) >= 0) break;
                __nanosleep(100);
                if ((++spins & 0x3Fu) == 0 && clock64() - t0 > 4000000000ll) {
                    good = 0;
                    atomicOr(a.status, 1024u);
                    break;
                }
            }
        }
        ok = good;
    }
    __syncthreads();
    // everything earlier in this stream has finished and is visible before out is written
    grid_dependency_wait();
    if (a.strict_release) grid_launch_dependents();
    if (!ok) return;
    const uint32_t D = a.head_dim;
    float mx = -1e30f;
    for (uint32_t r = 0; r < a.world; ++r)
        if (a.expected[r]) mx = fmaxf(mx, __ldcv(a.gather + r * a.block + (size_t)a.rows * D + row));
    float lt = 0.f;
    for (uint32_t r = 0; r < a.world; ++r) {
        if (!a.expected[r]) continue;
        const float ls = __ldcv(a.gather + r * a.block + (size_t)a.rows * D + a.rows + row);
        if (ls > 0.f) lt += ls * __expf(__ldcv(a.gather + r * a.block + (size_t)a.rows * D + row) - mx);
    }
    const float inv = ((fabsf(lt) <= 3.0e38f) && fabsf(lt) > 1e-6f) ? 1.0f / lt : 0.f;
    for (uint32_t d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.f;
        for (uint32_t r = 0; r < a.world; ++r) {
            if (!a.expected[r]) continue;
            acc += __ldcv(a.gather + r * a.block + (size_t)row * D + d) *
                   __expf(__ldcv(a.gather + r * a.block + (size_t)a.rows * D + row) - mx);
        }
        out[(size_t)row * D + d] = __float2half_rn(acc * inv);
    }
    __syncthreads();  // every thread of the block has consumed what it read from the receive blocks
    if (threadIdx.x < a.world && a.merged_dst[threadIdx.x]) atomicAdd_system(a.merged_dst[threadIdx.x], 1u);
}

}  // namespace
}  // namespace mf

using namespace mf;

extern "C" {

mf_status mf_peer_exchange_create(MfContext *ctx, uint32_t world, uint32_t rank, uint32_t rows, uint32_t head_dim,
                                  MfPeerExchange *px, uint8_t *handle_out)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!px) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "peer exchange: null");
    if (world == 0 || world > 8 || rank >= world || rows == 0 || head_dim == 0)
        return fail(ctx, MF_ERR_INVALID_OPERATION, "peer exchange: rank %u of %u, %u rows x %u", rank, world, rows, head_dim);
    memset(px, 0, sizeof(*px));
    // two step parities x world blocks of rows x (head_dim + 2) values, twice: as plain floats (the counted form), and
    // behind them as 8-byte words of a float and its tag (the tagged form)
    const size_t bytes = counter_bytes(rows) + (size_t)2 * world * rows * (head_dim + 2) * 3 * sizeof(float);
    void *base = nullptr;
    mf_status st = check_cuda(ctx, cudaMalloc(&base, bytes), "peer exchange: cudaMalloc");
    if (st != MF_OK) return st;
    st = check_cuda(ctx, cudaMemset(base, 0, bytes), "peer exchange: cudaMemset");
    if (st == MF_OK && handle_out) {
        cudaIpcMemHandle_t h;
        st = check_cuda(ctx, cudaIpcGetMemHandle(&h, base), "cudaIpcGetMemHandle");
        if (st == MF_OK) memcpy(handle_out, &h, sizeof(h));
    }
    if (st != MF_OK) {
        cudaFree(base);
        return st;
    }
    px->world = world;
    px->rank = rank;
    px->rows = rows;
    px->head_dim = head_dim;
    px->mapping[rank] = base;
    px->counters[rank] = static_cast<uint32_t *>(base);
    px->recv[rank] = reinterpret_cast<float *>(static_cast<char *>(base) + counter_bytes(rows));
    return MF_OK;
}

mf_status mf_peer_exchange_attach(MfContext *ctx, MfPeerExchange *px, uint32_t peer, const uint8_t *handle)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!px || !handle) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "peer exchange: null");
    if (peer >= px->world || peer == px->rank || px->mapping[peer])
        return fail(ctx, MF_ERR_INVALID_OPERATION, "peer exchange: cannot attach rank %u", peer);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void *base = nullptr;
    // opened in this context's device: the runtime enables peer access to the owner's GPU
    mf_status st = check_cuda(ctx, cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    if (st != MF_OK) return st;
    px->mapping[peer] = base;
    px->counters[peer] = static_cast<uint32_t *>(base);
    px->recv[peer] = reinterpret_cast<float *>(static_cast<char *>(base) + counter_bytes(px->rows));
    return MF_OK;
}

mf_status mf_peer_exchange_destroy(MfContext *ctx, MfPeerExchange *px)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!px) return MF_OK;
    cudaStreamSynchronize(ctx->stream);
    for (uint32_t r = 0; r < px->world && r < 8; ++r) {
        if (!px->mapping[r]) continue;
        if (r == px->rank) cudaFree(px->mapping[r]);
        else cudaIpcCloseMemHandle(px->mapping[r]);
    }
    memset(px, 0, sizeof(*px));
    return MF_OK;
}

// ---- the library-collective route: ncclAllGather of every rank's [acc | m | l] block, then the merge ----

mf_status mf_context_set_allgather(MfContext *ctx, MfAllGatherFn fn)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    ctx->allgather_fn = reinterpret_cast<void *>(fn);
    return MF_OK;
}

// ncclAllGather of the NCCL library this process already uses (or can load), bound at first use: the library
// itself does not link NCCL.
static int nccl_all_gather(const void *send, void *recv, uint64_t count_floats, void *comm, void *stream)
{
    typedef int (*Fn)(const void *, void *, size_t, int, void *, cudaStream_t);
    static Fn fn = nullptr;
    static bool looked = false;
    if (!looked) {
        looked = true;
        void *sym = dlsym(RTLD_DEFAULT, "ncclAllGather");
        if (!sym) {
            if (void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL)) sym = dlsym(h, "ncclAllGather");
        }
        fn = reinterpret_cast<Fn>(sym);
    }
    if (!fn) return -1;
    return fn(send, recv, (size_t)count_floats, 7 /* ncclFloat32 */, comm, static_cast<cudaStream_t>(stream));
}

mf_status mf_allgather_merge(MfContext *ctx, void *comm, const float *mine, float *gathered, uint32_t world, uint32_t rows,
                             uint32_t head_dim, void *out)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!mine || !gathered || !out) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "all-gather merge: null buffer");
    if (world == 0 || rows == 0 || head_dim == 0) return fail(ctx, MF_ERR_INVALID_OPERATION, "all-gather merge: world %u, rows %u", world, rows);
    const uint64_t block = (uint64_t)rows * (head_dim + 2);
    MfAllGatherFn fn = ctx->allgather_fn ? reinterpret_cast<MfAllGatherFn>(ctx->allgather_fn) : nccl_all_gather;
    if (!ctx->allgather_fn && !comm) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "all-gather merge: communicator");
    const int rc = fn(mine, gathered, block, comm, ctx->stream);
    if (rc != 0)
        return fail(ctx, MF_ERR_NCCL, rc == -1 && !ctx->allgather_fn ? "all-gather merge: ncclAllGather is not available in this process"
                                                                      : "all-gather merge: the all-gather failed (code %d)", rc);
    return mf_merge_partials_strided(ctx, gathered, gathered + (uint64_t)rows * head_dim, gathered + (uint64_t)rows * head_dim + rows,
                                     world, rows, head_dim, block, out);
}

mf_status mf_merge_pushed(MfContext *ctx, const MfPeerExchange *px, const uint32_t *units_per_rank, uint32_t step,
                          uint32_t rows, uint32_t head_dim, void *out)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (!px || !units_per_rank || !out) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "merge pushed: null input");
    if (px->world == 0 || px->world > 8 || px->rank >= px->world)
        return fail(ctx, MF_ERR_INVALID_OPERATION, "peer exchange: rank %u of %u", px->rank, px->world);
    if (rows == 0 || head_dim == 0) return MF_OK;
    if (rows != px->rows || head_dim != px->head_dim)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "merge pushed: the exchange was created for %u rows x %u, this call has %u x %u",
                    px->rows, px->head_dim, rows, head_dim);
    PushedMergeArgs a{};
    a.block = (uint64_t)rows * (head_dim + 2);
    a.gather = px->recv[px->rank] + (uint64_t)(step & 1) * px->world * a.block;
    a.counters = px->counters[px->rank];
    a.world = px->world;
    a.rows = rows;
    a.head_dim = head_dim;
    a.status = ctx->d_status;
    for (uint32_t r = 0; r < px->world; ++r) a.expected[r] = units_per_rank[r] * (step + 1);
    if (px->merge_only_mask >> px->rank & 1u) {
        if (units_per_rank[px->rank])
            return fail(ctx, MF_ERR_INVALID_OPERATION, "merge pushed: rank %u is in merge_only_mask but pushes %u units",
                        px->rank, units_per_rank[px->rank]);
        for (uint32_t r = 0; r < px->world; ++r)
            if (r != px->rank && px->counters[r]) a.merged_dst[r] = px->counters[r] + kPeerMergedBy + px->rank;
    }
    if (ctx->overlap_launches) {
        a.strict_release = ctx->next_launch_strict() ? 1u : 0u;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(rows);
        cfg.blockDim = dim3(128);
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, merge_pushed_kernel, a, static_cast<__half *>(out));
        if (e != cudaSuccess) return fail(ctx, MF_ERR_CUDA, "launch merge_pushed_kernel: %s", cudaGetErrorString(e));
        ++ctx->launches;
        ctx->note_programmatic_launch(a.strict_release != 0, nullptr, nullptr);
        return MF_OK;
    }
    merge_pushed_kernel<<<rows, 128, 0, ctx->stream>>>(a, static_cast<__half *>(out));
    return check_launch(ctx, "merge_pushed_kernel");
}

}  // extern "C"
