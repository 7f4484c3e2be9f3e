// Context, error reporting, scratch arena and tensor-map cache.
//
// MfContext stands in for the reference's Foundry object (src/lib.rs:57-353):
// one device, one in-order command stream, pooled scratch.  Metal pipeline
// compilation, argument binding and per-dispatch barriers have no counterpart:
// a CUDA stream already orders the launches.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "internal.hpp"

namespace mf {

mf_status fail(MfContext *ctx, mf_status code, const char *fmt, ...)
{
    if (ctx) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof(buf), fmt, ap);
        va_end(ap);
        ctx->last_error = buf;
    }
    return code;
}

mf_status check_cuda(MfContext *ctx, cudaError_t e, const char *what)
{
    if (e == cudaSuccess) return MF_OK;
    return fail(ctx, e == cudaErrorMemoryAllocation ? MF_ERR_OUT_OF_MEMORY : MF_ERR_CUDA, "%s: %s", what,
                cudaGetErrorString(e));
}

mf_status check_launch(MfContext *ctx, const char *what)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(ctx, MF_ERR_CUDA, "launch %s: %s", what, cudaGetErrorString(e));
    ++ctx->launches;
    return MF_OK;
}

mf_status need_tensor(MfContext *ctx, const MfTensor *t, const char *name)
{
    if (!t || !t->dev_ptr) return fail(ctx, MF_ERR_INPUT_NOT_FOUND, "%s", name);
    if (t->dtype != MF_DTYPE_F16) return fail(ctx, MF_ERR_UNSUPPORTED_DTYPE, "%s must be F16", name);
    if (t->rank == 0 || t->rank > 4) return fail(ctx, MF_ERR_INVALID_SHAPE, "%s: rank %u", name, t->rank);
    return MF_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

mf_status get_tensor_map(MfContext *ctx, const void *base, uint64_t rows, uint32_t cols, uint32_t box_rows,
                         uint32_t box_cols, CUtensorMap *out, uint32_t whole_rows)
{
    TensorMapKey key{base, rows, cols, box_rows, box_cols, whole_rows};
    auto it = ctx->tmaps.find(key);
    if (it != ctx->tmaps.end()) {
        *out = it->second;
        return MF_OK;
    }
    if (!ctx->encode_fn) {
        cudaDriverEntryPointQueryResult q;
        void *fn = nullptr;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
            return fail(ctx, MF_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
        ctx->encode_fn = fn;
    }
    if (reinterpret_cast<uintptr_t>(base) & 15u)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "K/V base pointer must be 16-byte aligned");
    if (box_cols * 2 != 128 || cols % box_cols != 0 || box_rows == 0 || box_rows > 256)
        return fail(ctx, MF_ERR_INVALID_SHAPE, "tensor-map box [%u x %u] unsupported", box_rows, box_cols);
    CUtensorMap tm;
    CUresult r;
    if (whole_rows) {
        if (cols != 128) return fail(ctx, MF_ERR_INVALID_SHAPE, "whole-row tensor map needs 128 columns");
        // (64 cols, rows, 2 halves): the half index is the OUTER box dimension so that shared
        // memory receives [half][rows][128 B]; its global stride (128 B) is smaller than the row
        // stride (256 B), which the address arithmetic of a tiled copy does not mind.
        cuuint64_t gdim[3] = {64, rows, 2};
        cuuint64_t gstride[2] = {256, 128};
        cuuint32_t box[3] = {64, box_rows, 2};
        cuuint32_t estr[3] = {1, 1, 1};
        r = reinterpret_cast<EncodeTiledFn>(ctx->encode_fn)(
            &tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(base), gdim, gstride, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        cuuint64_t gdim[2] = {cols, rows};
        cuuint64_t gstride[1] = {(cuuint64_t)cols * 2};
        cuuint32_t box[2] = {box_cols, box_rows};
        cuuint32_t estr[2] = {1, 1};
        r = reinterpret_cast<EncodeTiledFn>(ctx->encode_fn)(
            &tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), gdim, gstride, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) return fail(ctx, MF_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    if (ctx->tmaps.size() > 4096) ctx->tmaps.clear();
    ctx->tmaps.emplace(key, tm);
    *out = tm;
    return MF_OK;
}

mf_status ensure_scratch(MfContext *ctx, uint64_t bytes)
{
    if (ctx->scratch && ctx->scratch_bytes >= bytes) return MF_OK;
    if (ctx->scratch && !ctx->scratch_owned)
        return fail(ctx, MF_ERR_OUT_OF_MEMORY, "caller-provided scratch too small: need %llu bytes, have %llu",
                    (unsigned long long)bytes, (unsigned long long)ctx->scratch_bytes);
    if (ctx->scratch) {
        // Work already queued may still use the old arena.
        mf_status st = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
        if (st != MF_OK) return st;
        cudaFree(ctx->scratch);
        ctx->scratch = nullptr;
        ctx->scratch_bytes = 0;
    }
    uint64_t want = bytes < (8ull << 20) ? (8ull << 20) : bytes + bytes / 2;
    mf_status st = check_cuda(ctx, cudaMalloc(&ctx->scratch, want), "cudaMalloc(scratch)");
    if (st != MF_OK) return st;
    ctx->scratch_bytes = want;
    ctx->scratch_owned = true;
    return check_cuda(ctx, cudaMemsetAsync(ctx->scratch, 0, kCounterRegionBytes, ctx->stream),
                      "cudaMemsetAsync(scratch counters)");
}

}  // namespace mf

using namespace mf;

extern "C" {

uint32_t mf_abi_version(void) { return 1; }

const char *mf_status_name(mf_status s)
{
    switch (s) {
        case MF_OK: return "Ok";
        case MF_ERR_OPERATION_NOT_SUPPORTED: return "OperationNotSupported";
        case MF_ERR_INVALID_SHAPE: return "InvalidShape";
        case MF_ERR_INVALID_OPERATION: return "InvalidOperation";
        case MF_ERR_INPUT_NOT_FOUND: return "InputNotFound";
        case MF_ERR_UNSUPPORTED_DTYPE: return "UnsupportedDtype";
        case MF_ERR_OUT_OF_MEMORY: return "OutOfMemory";
        case MF_ERR_CUDA: return "CudaError";
        case MF_ERR_NCCL: return "NcclError";
        case MF_ERR_TIMEOUT: return "Timeout";
        default: return "Unknown";
    }
}

mf_status mf_context_create(int32_t device, void *cuda_stream, MfContext **out)
{
    if (!out) return MF_ERR_INPUT_NOT_FOUND;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) return MF_ERR_CUDA;  // no device: no fallback
    if (device < 0 || device >= n) return MF_ERR_INVALID_OPERATION;
    if (cudaSetDevice(device) != cudaSuccess) return MF_ERR_CUDA;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return MF_ERR_CUDA;
    if (prop.major != 10) return MF_ERR_OPERATION_NOT_SUPPORTED;  // built for sm_100a only
    MfContext *ctx = new MfContext();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    if (cuda_stream) {
        ctx->stream = static_cast<cudaStream_t>(cuda_stream);
    } else {
        if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
            delete ctx;
            return MF_ERR_CUDA;
        }
        ctx->own_stream = true;
    }
    if (cudaMalloc(reinterpret_cast<void **>(&ctx->d_status), 16) != cudaSuccess ||
        cudaMemset(ctx->d_status, 0, 16) != cudaSuccess) {
        mf_context_destroy(ctx);
        return MF_ERR_CUDA;
    }
    *out = ctx;
    return MF_OK;
}

void mf_context_destroy(MfContext *ctx)
{
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    if (ctx->scratch && ctx->scratch_owned) cudaFree(ctx->scratch);
    if (ctx->qkv_xn) cudaFree(ctx->qkv_xn);
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->own_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

mf_status mf_context_set_stream(MfContext *ctx, void *cuda_stream)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (ctx->own_stream && ctx->stream) {
        cudaStreamSynchronize(ctx->stream);
        cudaStreamDestroy(ctx->stream);
        ctx->own_stream = false;
    }
    ctx->stream = static_cast<cudaStream_t>(cuda_stream);
    return MF_OK;
}

mf_status mf_context_set_scratch(MfContext *ctx, void *dev_ptr, uint64_t bytes)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    if (dev_ptr && bytes < kCounterRegionBytes + (1u << 20))
        return fail(ctx, MF_ERR_INVALID_OPERATION, "scratch must be at least %u bytes",
                    kCounterRegionBytes + (1u << 20));
    if (ctx->scratch && ctx->scratch_owned) {
        cudaStreamSynchronize(ctx->stream);
        cudaFree(ctx->scratch);
    }
    ctx->scratch = dev_ptr;
    ctx->scratch_bytes = dev_ptr ? bytes : 0;
    ctx->scratch_owned = false;
    if (dev_ptr)
        return check_cuda(ctx, cudaMemsetAsync(dev_ptr, 0, kCounterRegionBytes, ctx->stream),
                          "cudaMemsetAsync(scratch counters)");
    return MF_OK;
}

mf_status mf_context_set_option(MfContext *ctx, uint32_t option, uint32_t value)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    switch (option) {
        case MF_OPTION_OVERLAP_LAUNCHES: ctx->overlap_launches = value > 2 ? 1u : value; return MF_OK;
        case MF_OPTION_DECODE_STAGES: ctx->decode_stages = value; return MF_OK;
        case MF_OPTION_PREFILL_IMPL: ctx->prefill_impl = value; return MF_OK;
        case MF_OPTION_QKV_IMPL: ctx->qkv_impl = value; return MF_OK;
        case MF_OPTION_PUSH_TAGGED: ctx->push_tagged = value ? 1u : 0u; return MF_OK;
        case MF_OPTION_PLAN_ITEM_COST: ctx->plan_item_cost = value ? value : mf::kPlanItemCost; return MF_OK;
        case MF_OPTION_DECODE_CLUSTERS: ctx->decode_clusters = value ? 1u : 0u; return MF_OK;
        default: return fail(ctx, MF_ERR_INVALID_OPERATION, "unknown option %u", option);
    }
}

mf_status mf_synchronize(MfContext *ctx)
{
    if (!ctx) return MF_ERR_INPUT_NOT_FOUND;
    mf_status st = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
    if (st != MF_OK) return st;
    uint32_t flag = 0;
    st = check_cuda(ctx, cudaMemcpy(&flag, ctx->d_status, 4, cudaMemcpyDeviceToHost), "read status");
    if (st != MF_OK) return st;
    if (flag) {
        cudaMemset(ctx->d_status, 0, 4);
        if (flag & ~kStatusBadPage) {
            if (ctx->scratch) cudaMemset(ctx->scratch, 0, kCounterRegionBytes);
            return fail(ctx, MF_ERR_TIMEOUT, "a device-side barrier wait ran out (status 0x%x)", flag);
        }
        return fail(ctx, MF_ERR_INVALID_OPERATION,
                    "a cache access was skipped: a page id outside the pool, or a position outside the page table, "
                    "in the caller's device-side table or lengths (status 0x%x)", flag);
    }
    return MF_OK;
}

const char *mf_last_error(const MfContext *ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }

uint64_t mf_launch_count(const MfContext *ctx) { return ctx ? ctx->launches : 0; }

}  // extern "C"
