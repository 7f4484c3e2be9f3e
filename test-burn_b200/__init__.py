"""Python host binding of libmetallic_cuda.so (the C ABI in include/metallic_cuda.h).

The names follow the metallic-foundry operator layer this library stands in for
(crates/metallic-foundry/src/metals/{kv_prep,sdpa,flashattention,rope,kv_cache_write}):
`Foundry` (context), `KvPrepFused`, `FlashAttentionStep`, `run_flash_decode`,
`RopeFlashDecodeStep`, `KvCacheWrite`, `KvCacheRead`, `Rope`, plus the paged
batched-decode entry points, which the reference does not have.

There is no fallback path: importing works without a GPU (so that the symbol table
can be checked), but creating a `Foundry` raises `MetalError` when no sm_100
device is present, and a missing shared library raises at import.

PyTorch appears here only as the owner of device buffers and streams; the shared
library itself does not link it.
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
from pathlib import Path

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "libmetallic_cuda.so"
if not _SO.exists():
    raise ImportError(f"{_SO} is missing: build it with `python {_HERE / 'build.py'}` (no CPU fallback exists)")
lib = C.CDLL(str(_SO))

u32 = C.c_uint32
u64 = C.c_uint64
vp = C.c_void_p

MF_OK = 0
STATUS_NAMES = {0: "Ok", 1: "OperationNotSupported", 2: "InvalidShape", 3: "InvalidOperation", 4: "InputNotFound",
                5: "UnsupportedDtype", 6: "OutOfMemory", 7: "CudaError", 8: "NcclError", 9: "Timeout"}
ROPE_MODE_NEOX, ROPE_MODE_NORMAL = 0, 1
ROUTE_DECODE, ROUTE_PREFILL, ROUTE_PREFILL_SPLITK, ROUTE_REFERENCE = 1, 2, 3, 4
DTYPE_F16, DTYPE_F32, DTYPE_U32 = 0, 1, 2
ALL_SEQUENCES = 0xFFFFFFFF
OPTION_OVERLAP_LAUNCHES, OPTION_DECODE_STAGES, OPTION_PREFILL_IMPL, OPTION_DECODE_CLUSTERS, OPTION_QKV_IMPL = 1, 2, 3, 4, 5
OPTION_PLAN_ITEM_COST = 6
OPTION_PUSH_TAGGED = 7
KV_LAYOUT_EXPANDED_HEADS, KV_LAYOUT_COMPACT_KV_HEADS = 0, 1


ALLGATHER_FN = C.CFUNCTYPE(C.c_int, vp, vp, u64, vp, vp)


class MetalError(RuntimeError):
    """Raised for any non-zero mf_status; `.kind` is the MetalError variant name."""

    def __init__(self, status: int, message: str):
        self.status = status
        self.kind = STATUS_NAMES.get(status, "Unknown")
        super().__init__(f"{self.kind}: {message}")


class MfTensor(C.Structure):
    _fields_ = [("dev_ptr", vp), ("offset_bytes", u64), ("dtype", u32), ("rank", u32), ("dims", u64 * 4),
                ("strides", u64 * 4)]


def _u32_struct(name, fields):
    return type(name, (C.Structure,), {"_fields_": [(f, u32) for f in fields]})


KvPrepFusedParamsResolved = _u32_struct("KvPrepFusedParamsResolved", (
    "d_model", "kv_dim", "head_dim", "n_heads", "n_kv_heads", "group_size", "seq_len", "position_offset",
    "max_seq_len", "total_elements", "rope_mode", "layer_idx", "no_rope_layer_step"))
RopeParamsResolved = _u32_struct("RopeParamsResolved", ("dim", "seq_len", "position_offset", "total_elements"))
KvCacheWriteParamsResolved = _u32_struct("KvCacheWriteParamsResolved", (
    "n_kv_heads", "head_dim", "input_seq_len", "position_offset", "max_seq_len", "total_elements", "layer_idx"))
KvCacheWriteRepeatKvHeadsParamsResolved = _u32_struct("KvCacheWriteRepeatKvHeadsParamsResolved", (
    "n_kv_heads", "n_heads", "group_size", "head_dim", "input_seq_len", "position_offset", "max_seq_len",
    "total_elements", "layer_idx"))
MfFlashDecodeStrides = _u32_struct("MfFlashDecodeStrides", (
    "q_stride_b", "q_stride_h", "k_stride_b", "k_stride_h", "v_stride_b", "v_stride_h", "out_stride_b",
    "out_stride_h"))
MfFlashAttentionArgs = _u32_struct("MfFlashAttentionArgs", (
    "causal", "query_offset", "n_heads", "head_dim", "kv_seq_len", "m", "kv_head_major"))


class SdpaParams(C.Structure):
    _fields_ = [("kv_len", u32), ("head_dim", u32), ("scale", C.c_float), ("stride_k_s", u32), ("stride_v_s", u32)]


class SdpaPrefillParams(C.Structure):
    _fields_ = [("kv_len", u32), ("head_dim", u32), ("scale", C.c_float)] + [(f, u32) for f in (
        "stride_k_s", "stride_v_s", "query_offset", "q_stride_b", "q_stride_h", "k_stride_b", "k_stride_h",
        "v_stride_b", "v_stride_h", "out_stride_b", "out_stride_h", "q_stride_m", "out_stride_m", "group_size",
        "q_len")]


class SdpaPrefillSplitKParams(C.Structure):
    _fields_ = [("base", SdpaPrefillParams), ("n_heads", u32), ("split_k", u32)]


class MfKvGeometry(C.Structure):
    _fields_ = [(f, u32) for f in ("n_heads", "n_kv_heads", "group_size", "head_dim", "layout", "cache_heads")]


class MfContextConfig(C.Structure):
    _fields_ = [("max_context_len", u64), ("allocated_capacity", u64), ("budget_bytes", u64), ("budget_auto_pct", C.c_float),
                ("full_reserve", u32)]


class MfPagedKv(C.Structure):
    _fields_ = [("k_pool", vp), ("v_pool", vp), ("page_table", vp), ("kv_lens", vp), ("n_pages", u32),
                ("n_kv_heads", u32), ("page_size", u32), ("head_dim", u32), ("page_table_stride", u32),
                ("batch", u32)]


class MfPagedKv8(C.Structure):
    _fields_ = [("k_pool", vp), ("v_pool", vp), ("k_scales", vp), ("v_scales", vp), ("page_table", vp), ("kv_lens", vp),
                ("n_pages", u32), ("n_kv_heads", u32), ("page_size", u32), ("head_dim", u32), ("page_table_stride", u32),
                ("batch", u32)]


class KvRearrangeParamsResolved(C.Structure):
    _fields_ = [(n, u32) for n in ("kv_dim", "row_stride", "kv_head_dim", "n_heads", "n_kv_heads", "head_dim", "seq",
                                   "total_elements")]


class RepeatKvHeadsParamsResolved(C.Structure):
    _fields_ = [(n, u32) for n in ("group_size", "batch", "n_kv_heads", "n_heads", "seq", "head_dim", "cache_stride",
                                   "total_elements")]


class MfPagedDecodeArgs(C.Structure):
    _fields_ = [("q", vp), ("k", vp), ("v", vp), ("q_rot", vp), ("out", vp), ("cos", vp), ("sin", vp),
                ("n_heads", u32), ("rope", u32), ("rope_mode", u32), ("append", u32), ("scale", C.c_float)]


class MfPagedPrefillArgs(C.Structure):
    _fields_ = [("q", vp), ("out", vp), ("seq", u32), ("q_len", u32), ("kv_len", u32), ("query_offset", u32),
                ("n_heads", u32), ("q_stride_h", u32), ("q_stride_m", u32), ("out_stride_h", u32), ("out_stride_m", u32),
                ("scale", C.c_float)]


class MfFusedQkvArgs(C.Structure):
    _fields_ = [("input", vp), ("w_q", vp), ("w_k", vp), ("w_v", vp), ("gamma", vp), ("bias_q", vp), ("bias_k", vp),
                ("bias_v", vp), ("out_q", vp), ("out_k", vp), ("out_v", vp), ("k_dim", u32), ("n_dim", u32),
                ("n_kv", u32), ("m", u32), ("weights_per_block", u32), ("epsilon", C.c_float)]


class MfPeerExchange(C.Structure):
    _fields_ = [("recv", vp * 8), ("counters", vp * 8), ("mapping", vp * 8), ("world", u32), ("rank", u32),
                ("rows", u32), ("head_dim", u32), ("merge_only_mask", u32)]


# Every symbol declared in include/metallic_cuda.h, with its signature.
_SIGNATURES = {
    "mf_context_create": (C.c_int32, [C.c_int32, vp, C.POINTER(vp)]),
    "mf_context_destroy": (None, [vp]),
    "mf_context_set_stream": (C.c_int32, [vp, vp]),
    "mf_synchronize": (C.c_int32, [vp]),
    "mf_last_error": (C.c_char_p, [vp]),
    "mf_status_name": (C.c_char_p, [C.c_int32]),
    "mf_abi_version": (u32, []),
    "mf_launch_count": (u64, [vp]),
    "mf_context_set_scratch": (C.c_int32, [vp, vp, u64]),
    "mf_context_set_option": (C.c_int32, [vp, u32, u32]),
    "mf_rope_tables_host": (C.c_int32, [C.c_float, u32, u32, u32, vp, vp, vp]),
    "mf_align_capacity": (u64, [u64]),
    "mf_grown_capacity": (u64, [u64, u64, u64]),
    "mf_kv_per_token_bytes_f16": (u64, [u32, u32, u32]),
    "mf_estimate_kv_memory": (u64, [u32, u32, u32, u64]),
    "mf_prefill_split_k": (u32, [u32, u32]),
    "mf_kv_geometry_from_architecture": (C.c_int32, [u32, u32, u32, C.POINTER(MfKvGeometry)]),
    "mf_kv_geometry_from_cache_tensor": (C.c_int32, [u32, u32, u32, C.POINTER(MfTensor), u64, C.POINTER(MfKvGeometry),
                                                     C.c_char_p, u32]),
    "mf_context_config_from_architecture": (C.c_int32, [u64, u64, u64, u32, C.c_int64, C.POINTER(MfContextConfig)]),
    "mf_context_config_from_env": (C.c_int32, [u64, u64, C.POINTER(MfContextConfig)]),
    "mf_apply_memory_budget": (C.c_int32, [C.POINTER(MfContextConfig), u64, u64]),
    "mf_kv_prep_fused": (C.c_int32, [vp] + [C.POINTER(MfTensor)] * 8 + [C.POINTER(KvPrepFusedParamsResolved)]),
    "mf_rope": (C.c_int32, [vp] + [C.POINTER(MfTensor)] * 4 + [C.POINTER(RopeParamsResolved)]),
    "mf_kv_cache_write": (C.c_int32, [vp, C.POINTER(MfTensor), C.POINTER(MfTensor),
                                      C.POINTER(KvCacheWriteParamsResolved)]),
    "mf_kv_cache_write_repeat_kv_heads": (C.c_int32, [vp, C.POINTER(MfTensor), C.POINTER(MfTensor),
                                                      C.POINTER(KvCacheWriteRepeatKvHeadsParamsResolved)]),
    "mf_kv_cache_read": (C.c_int32, [vp, C.POINTER(MfTensor), C.POINTER(MfTensor), u32]),
    "mf_kv_cache_grow": (C.c_int32, [vp, C.POINTER(MfTensor), C.POINTER(MfTensor), u32]),
    "mf_kv_cache_to_pages": (C.c_int32, [vp, C.POINTER(MfTensor), C.POINTER(MfPagedKv), u32, u32, u32]),
    "mf_kv_rearrange": (C.c_int32, [vp, C.POINTER(MfTensor), C.POINTER(MfTensor), C.POINTER(KvRearrangeParamsResolved)]),
    "mf_repeat_kv_heads": (C.c_int32, [vp, C.POINTER(MfTensor), C.POINTER(MfTensor),
                                       C.POINTER(RepeatKvHeadsParamsResolved)]),
    "mf_sdpa_reference": (C.c_int32, [vp] + [C.POINTER(MfTensor)] * 4 + [C.POINTER(MfFlashAttentionArgs)]),
    "mf_flash_attention": (C.c_int32, [vp] + [C.POINTER(MfTensor)] * 4 + [C.POINTER(MfFlashAttentionArgs),
                                                                         C.POINTER(u32)]),
    "mf_run_flash_decode": (C.c_int32, [vp] + [C.POINTER(MfTensor)] * 4 + [u32] * 5),
    "mf_flash_decode": (C.c_int32, [vp, vp, vp, vp, vp, C.POINTER(MfFlashDecodeStrides), C.POINTER(SdpaParams),
                                    u32, u32, u32]),
    "mf_flash_decode_static_scratch": (C.c_int32, [vp, vp, vp, vp, vp, C.POINTER(MfFlashDecodeStrides),
                                                   C.POINTER(SdpaParams), u32, u32, C.c_char_p, u32]),
    "mf_static_scratch_status": (C.c_int32, [vp, C.POINTER(u32)]),
    "mf_rope_flash_decode": (C.c_int32, [vp, vp, vp, vp, vp, vp, vp, C.POINTER(RopeParamsResolved),
                                         C.POINTER(SdpaParams), C.POINTER(MfFlashDecodeStrides), u32, u32]),
    "mf_flash_prefill": (C.c_int32, [vp, vp, vp, vp, vp, C.POINTER(SdpaPrefillSplitKParams)]),
    "mf_merge_partials": (C.c_int32, [vp, vp, vp, vp, u32, u32, u32, vp]),
    "mf_merge_partials_strided": (C.c_int32, [vp, vp, vp, vp, u32, u32, u32, u64, vp]),
    "mf_decode_plan_create": (C.c_int32, [vp, vp, u32, u32, u32, u32, u32, u32, C.POINTER(vp)]),
    "mf_decode_plan_update": (C.c_int32, [vp, vp, vp]),
    "mf_decode_plan_destroy": (None, [vp, vp]),
    "mf_decode_plan_build_host": (u32, [vp, u32, u32, u32, vp, u32, vp, C.POINTER(u32)]),
    "mf_decode_plan_build_host_clusters": (u32, [vp, u32, u32, u32, u32, u32, u32, vp, u32, C.POINTER(u32), C.POINTER(u32)]),
    "mf_decode_plan_ctas": (u32, [vp]),
    "mf_decode_plan_cluster": (u32, [vp]),
    "mf_decode_plan_items": (u32, [vp]),
    "mf_decode_plan_tiles": (u64, [vp]),
    "mf_paged_decode": (C.c_int32, [vp, vp, C.POINTER(MfPagedKv), C.POINTER(MfPagedDecodeArgs)]),
    "mf_paged_decode_kv8": (C.c_int32, [vp, vp, C.POINTER(MfPagedKv8), C.POINTER(MfPagedDecodeArgs)]),
    "mf_paged_prefill_kv8_workspace_bytes": (C.c_uint64, [C.POINTER(MfPagedKv8), C.c_uint32]),
    "mf_paged_prefill_kv8": (C.c_int32, [vp, C.POINTER(MfPagedKv8), C.POINTER(MfPagedPrefillArgs), vp, C.c_uint64]),
    "mf_paged_decode_kv8_partial_push": (C.c_int32, [vp, vp, C.POINTER(MfPagedKv8), C.POINTER(MfPagedDecodeArgs), vp,
                                                     C.POINTER(MfPeerExchange), C.c_uint32]),
    "mf_paged_decode_kv8_push_merge": (C.c_int32, [vp, vp, C.POINTER(MfPagedKv8), C.POINTER(MfPagedDecodeArgs), vp,
                                                   C.POINTER(MfPeerExchange), C.c_uint32, C.c_uint32]),
    "mf_paged_decode_kv8_partial": (C.c_int32, [vp, vp, C.POINTER(MfPagedKv8), C.POINTER(MfPagedDecodeArgs), vp, vp, vp, vp]),
    "mf_paged_kv8_append": (C.c_int32, [vp, C.POINTER(MfPagedKv8), vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32]),
    "mf_paged_kv8_gather": (C.c_int32, [vp, C.POINTER(MfPagedKv8), u32, u32, u32, vp]),
    "mf_paged_kv_append": (C.c_int32, [vp, C.POINTER(MfPagedKv), vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32,
                                       u32]),
    "mf_paged_gather": (C.c_int32, [vp, C.POINTER(MfPagedKv), u32, u32, u32, vp]),
    "mf_kv_prep_flash_decode": (C.c_int32, [vp] + [C.POINTER(MfTensor)] * 9 + [C.POINTER(KvPrepFusedParamsResolved)]),
    "mf_fused_qkv": (C.c_int32, [vp, C.POINTER(MfFusedQkvArgs)]),
    "mf_fused_qkv_kv_prep": (C.c_int32, [vp, C.POINTER(MfFusedQkvArgs)] + [C.POINTER(MfTensor)] * 5 +
                             [C.POINTER(KvPrepFusedParamsResolved)]),
    "mf_fused_qkv_paged_append": (C.c_int32, [vp, C.POINTER(MfFusedQkvArgs), C.POINTER(MfPagedKv), vp, vp, vp, u32, u32,
                                              u32, u32, u32]),
    "mf_paged_decode_partial_push": (C.c_int32, [vp, vp, C.POINTER(MfPagedKv), C.POINTER(MfPagedDecodeArgs), vp,
                                                 C.POINTER(MfPeerExchange), u32]),
    "mf_page_pool_create": (C.c_int32, [u32, C.POINTER(vp)]),
    "mf_page_pool_destroy": (None, [vp]),
    "mf_page_pool_alloc": (C.c_int32, [vp, u32, vp]),
    "mf_page_pool_retain": (C.c_int32, [vp, vp, u32]),
    "mf_page_pool_release": (C.c_int32, [vp, vp, u32]),
    "mf_page_pool_free_count": (u32, [vp]),
    "mf_page_pool_refcount": (u32, [vp, u32]),
    "mf_prefix_cache_default_entries": (u32, []),
    "mf_prefix_cache_create": (C.c_int32, [vp, u32, u32, C.POINTER(vp)]),
    "mf_prefix_cache_destroy": (None, [vp]),
    "mf_prefix_cache_entries": (u32, [vp]),
    "mf_prefix_cache_store": (C.c_int32, [vp, vp, u32, C.c_char_p, vp, u32]),
    "mf_prefix_cache_lookup": (C.c_int32, [vp, vp, u32, C.c_char_p, C.POINTER(u32), vp, u32, C.POINTER(u32)]),
    "mf_paged_prefill": (C.c_int32, [vp, C.POINTER(MfPagedKv), C.POINTER(MfPagedPrefillArgs)]),
    "mf_paged_copy_pages": (C.c_int32, [vp, C.POINTER(MfPagedKv), vp, vp, u32]),
    "mf_peer_exchange_create": (C.c_int32, [vp, u32, u32, u32, u32, C.POINTER(MfPeerExchange), vp]),
    "mf_peer_exchange_attach": (C.c_int32, [vp, C.POINTER(MfPeerExchange), u32, vp]),
    "mf_peer_exchange_destroy": (C.c_int32, [vp, C.POINTER(MfPeerExchange)]),
    "mf_paged_decode_push_merge": (C.c_int32, [vp, vp, C.POINTER(MfPagedKv), C.POINTER(MfPagedDecodeArgs), vp,
                                               C.POINTER(MfPeerExchange), u32, u32]),
    "mf_allgather_merge": (C.c_int32, [vp, vp, vp, vp, u32, u32, u32, vp]),
    "mf_context_set_allgather": (C.c_int32, [vp, vp]),
    "mf_merge_pushed": (C.c_int32, [vp, C.POINTER(MfPeerExchange), vp, u32, u32, u32, vp]),
    "mf_paged_decode_partial": (C.c_int32, [vp, vp, C.POINTER(MfPagedKv), C.POINTER(MfPagedDecodeArgs), vp, vp, vp,
                                            vp]),
}
for _name, (_res, _args) in _SIGNATURES.items():
    _fn = getattr(lib, _name)  # AttributeError here means the library does not export a declared symbol
    _fn.restype = _res
    _fn.argtypes = _args

EXPORTED_SYMBOLS = tuple(_SIGNATURES)


def tensor_arg(t, dims=None, strides=None) -> MfTensor:
    """TensorArg::from_tensor for a torch tensor (dims/strides may be overridden to
    describe metadata that differs from the buffer's true layout, as the reference does
    for q_rot)."""
    import torch

    dt = {torch.float16: DTYPE_F16, torch.float32: DTYPE_F32, torch.int32: DTYPE_U32, torch.uint32: DTYPE_U32}
    if t.dtype not in dt:
        code = 99
    else:
        code = dt[t.dtype]
    dims = list(t.shape) if dims is None else list(dims)
    strides = list(t.stride()) if strides is None else list(strides)
    m = MfTensor()
    m.dev_ptr = t.data_ptr()
    m.offset_bytes = 0
    m.dtype = code
    m.rank = len(dims)
    for i, (d, s) in enumerate(zip(dims, strides)):
        m.dims[i] = d
        m.strides[i] = s
    return m


def _ptr(t):
    return None if t is None else t.data_ptr()


class Foundry:
    """Device + in-order stream + scratch (Foundry, src/lib.rs:57-353)."""

    def __init__(self, device: int = 0, stream=None):
        h = vp()
        stream_ptr = None if stream is None else int(stream)
        st = lib.mf_context_create(device, stream_ptr, C.byref(h))
        if st != MF_OK:
            raise MetalError(st, "mf_context_create failed (no sm_100 CUDA device? there is no CPU fallback)")
        self._h = h
        self.device = device

    def close(self):
        if getattr(self, "_h", None):
            lib.mf_context_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, st: int):
        if st != MF_OK:
            raise MetalError(st, (lib.mf_last_error(self._h) or b"").decode())

    def set_stream(self, stream):
        self.check(lib.mf_context_set_stream(self._h, None if stream is None else int(stream)))

    def synchronize(self):
        self.check(lib.mf_synchronize(self._h))

    def set_option(self, option: int, value: int):
        self.check(lib.mf_context_set_option(self._h, option, value))

    @property
    def launch_count(self) -> int:
        return int(lib.mf_launch_count(self._h))

    # -- operators -------------------------------------------------------------------------

    def kv_prep_fused(self, q, k, v, q_rot, k_cache, v_cache, cos, sin, params: KvPrepFusedParamsResolved):
        """foundry.run(&KvPrepFused{..}) (src/metals/kv_prep/mod.rs:157-182)."""
        ts = [tensor_arg(x) for x in (q, k, v, q_rot, k_cache, v_cache, cos, sin)]
        self.check(lib.mf_kv_prep_fused(self._h, *[C.byref(t) for t in ts], C.byref(params)))

    def kv_prep_flash_decode(self, q, k, v, q_rot, k_cache, v_cache, cos, sin, output, params: KvPrepFusedParamsResolved):
        """KvPrepFused and FlashAttention (decode route) in one launch; q_rot may be None."""
        ts = [None if x is None else tensor_arg(x) for x in (q, k, v, q_rot, k_cache, v_cache, cos, sin, output)]
        self.check(lib.mf_kv_prep_flash_decode(self._h, *[None if t is None else C.byref(t) for t in ts], C.byref(params)))

    def rope(self, x, out, cos, sin, params: RopeParamsResolved):
        ts = [tensor_arg(t) for t in (x, out, cos, sin)]
        self.check(lib.mf_rope(self._h, *[C.byref(t) for t in ts], C.byref(params)))

    def kv_cache_write(self, x, cache, params):
        a, b = tensor_arg(x), tensor_arg(cache)
        fn = lib.mf_kv_cache_write if isinstance(params, KvCacheWriteParamsResolved) \
            else lib.mf_kv_cache_write_repeat_kv_heads
        self.check(fn(self._h, C.byref(a), C.byref(b), C.byref(params)))

    def kv_cache_read(self, cache, out, seq_len: int):
        a, b = tensor_arg(cache), tensor_arg(out)
        self.check(lib.mf_kv_cache_read(self._h, C.byref(a), C.byref(b), seq_len))

    def kv_cache_grow(self, old_cache, new_cache, current_pos: int):
        """preserve_kv_cache of reallocate_kv_buffers (src/model/executor.rs:2437-2513)."""
        a, b = tensor_arg(old_cache), tensor_arg(new_cache)
        self.check(lib.mf_kv_cache_grow(self._h, C.byref(a), C.byref(b), current_pos))

    def kv_cache_to_pages(self, cache, paged: MfPagedKv, use_v: bool, seq: int, length: int):
        a = tensor_arg(cache)
        self.check(lib.mf_kv_cache_to_pages(self._h, C.byref(a), C.byref(paged), int(use_v), seq, length))

    def flash_attention(self, q, k, v, output, *, causal, query_offset, n_heads, head_dim, kv_seq_len, m=1,
                        kv_head_major=True, q_meta=None, out_meta=None) -> int:
        """FlashAttentionStep::execute (src/metals/sdpa/step.rs:160-503).  Returns the route."""
        args = MfFlashAttentionArgs(int(causal), query_offset, n_heads, head_dim, kv_seq_len, m, int(kv_head_major))
        tq = tensor_arg(q, *(q_meta or (None, None)))
        to = tensor_arg(output, *(out_meta or (None, None)))
        tk, tv = tensor_arg(k), tensor_arg(v)
        route = u32(0)
        self.check(lib.mf_flash_attention(self._h, C.byref(tq), C.byref(tk), C.byref(tv), C.byref(to), C.byref(args),
                                          C.byref(route)))
        return route.value

    def kv_rearrange(self, input, output, params: KvRearrangeParamsResolved):
        ti, to = tensor_arg(input), tensor_arg(output)
        self.check(lib.mf_kv_rearrange(self._h, C.byref(ti), C.byref(to), C.byref(params)))

    def repeat_kv_heads(self, input, output, params: RepeatKvHeadsParamsResolved):
        ti, to = tensor_arg(input), tensor_arg(output)
        self.check(lib.mf_repeat_kv_heads(self._h, C.byref(ti), C.byref(to), C.byref(params)))

    def sdpa_reference(self, q, k, v, output, *, causal, query_offset, n_heads, head_dim, kv_seq_len, m=1, q_meta=None,
                       out_meta=None):
        """SdpaReferenceStep (src/metals/sdpa/step.rs:89-158): attention with the general mask."""
        args = MfFlashAttentionArgs(int(causal), query_offset, n_heads, head_dim, kv_seq_len, m, 1)
        tq = tensor_arg(q, *(q_meta or (None, None)))
        to = tensor_arg(output, *(out_meta or (None, None)))
        tk, tv = tensor_arg(k), tensor_arg(v)
        self.check(lib.mf_sdpa_reference(self._h, C.byref(tq), C.byref(tk), C.byref(tv), C.byref(to), C.byref(args)))

    def run_flash_decode(self, q, k, v, output, n_heads, head_dim, kv_seq_len, q_seq_len=1, kv_head_major=True,
                         q_meta=None, out_meta=None):
        tq = tensor_arg(q, *(q_meta or (None, None)))
        to = tensor_arg(output, *(out_meta or (None, None)))
        tk, tv = tensor_arg(k), tensor_arg(v)
        self.check(lib.mf_run_flash_decode(self._h, C.byref(tq), C.byref(tk), C.byref(tv), C.byref(to), n_heads,
                                           head_dim, kv_seq_len, q_seq_len, int(kv_head_major)))

    def flash_decode(self, q, k, v, output, strides: MfFlashDecodeStrides, params: SdpaParams, n_heads, batch=1,
                     n_splits=0):
        self.check(lib.mf_flash_decode(self._h, _ptr(q), _ptr(k), _ptr(v), _ptr(output), C.byref(strides),
                                       C.byref(params), n_heads, batch, n_splits))

    def rope_flash_decode(self, q, k, v, cos, sin, output, rope: RopeParamsResolved, params: SdpaParams,
                          strides: MfFlashDecodeStrides, n_heads, batch=1):
        """RopeFlashDecodeStep (src/metals/flashattention/step.rs:54-306)."""
        self.check(lib.mf_rope_flash_decode(self._h, _ptr(q), _ptr(k), _ptr(v), _ptr(cos), _ptr(sin), _ptr(output),
                                            C.byref(rope), C.byref(params), C.byref(strides), n_heads, batch))

    def flash_prefill(self, q, k, v, output, params: SdpaPrefillSplitKParams):
        self.check(lib.mf_flash_prefill(self._h, _ptr(q), _ptr(k), _ptr(v), _ptr(output), C.byref(params)))

    def merge_partials(self, acc, m, l, out):
        n_splits, rows, d = acc.shape
        self.check(lib.mf_merge_partials(self._h, _ptr(acc), _ptr(m), _ptr(l), n_splits, rows, d, _ptr(out)))

    def merge_gathered(self, gathered, rows, head_dim, out):
        """Merge an all-gathered [world, rows*(head_dim+2)] f32 buffer of [acc | m | l] blocks."""
        world = gathered.shape[0]
        block = rows * (head_dim + 2)
        base = gathered.data_ptr()
        self.check(lib.mf_merge_partials_strided(self._h, base, base + rows * head_dim * 4,
                                                 base + (rows * head_dim + rows) * 4, world, rows, head_dim, block,
                                                 _ptr(out)))

    # -- paged cache -----------------------------------------------------------------------

    def decode_plan(self, kv_lens_host, *, n_heads, n_kv_heads, head_dim, page_size, max_ctas=0) -> "DecodePlan":
        return DecodePlan(self, kv_lens_host, n_heads, n_kv_heads, head_dim, page_size, max_ctas)

    def paged_decode(self, plan: "DecodePlan", cache: MfPagedKv, q, out, *, n_heads, scale=None, k=None, v=None,
                     cos=None, sin=None, rope=False, rope_mode=ROPE_MODE_NEOX, append=False, q_rot=None):
        scale = 1.0 / math.sqrt(cache.head_dim) if scale is None else scale
        a = MfPagedDecodeArgs(_ptr(q), _ptr(k), _ptr(v), _ptr(q_rot), _ptr(out), _ptr(cos), _ptr(sin), n_heads,
                              int(rope), rope_mode, int(append), scale)
        self.check(lib.mf_paged_decode(self._h, plan._h, C.byref(cache), C.byref(a)))

    def paged_decode_partial(self, plan, cache, q, acc, m, l, *, n_heads, rope_positions=None, scale=None, k=None,
                             v=None, cos=None, sin=None, rope=False, rope_mode=ROPE_MODE_NEOX, append=False):
        scale = 1.0 / math.sqrt(cache.head_dim) if scale is None else scale
        a = MfPagedDecodeArgs(_ptr(q), _ptr(k), _ptr(v), None, None, _ptr(cos), _ptr(sin), n_heads, int(rope),
                              rope_mode, int(append), scale)
        self.check(lib.mf_paged_decode_partial(self._h, plan._h, C.byref(cache), C.byref(a), _ptr(rope_positions),
                                               _ptr(acc), _ptr(m), _ptr(l)))

    def paged_decode_partial_push(self, plan, cache, q, px: MfPeerExchange, step: int, *, n_heads, rope_positions=None,
                                  scale=None, k=None, v=None, cos=None, sin=None, rope=False,
                                  rope_mode=ROPE_MODE_NEOX, append=False):
        scale = 1.0 / math.sqrt(cache.head_dim) if scale is None else scale
        a = MfPagedDecodeArgs(_ptr(q), _ptr(k), _ptr(v), None, None, _ptr(cos), _ptr(sin), n_heads, int(rope),
                              rope_mode, int(append), scale)
        self.check(lib.mf_paged_decode_partial_push(self._h, plan._h, C.byref(cache), C.byref(a), _ptr(rope_positions),
                                                    C.byref(px), step))

    def peer_exchange_create(self, world: int, rank: int, rows: int, head_dim: int):
        """Returns (MfPeerExchange, handle bytes to hand to the other ranks)."""
        px = MfPeerExchange()
        handle = (C.c_uint8 * 64)()
        self.check(lib.mf_peer_exchange_create(self._h, world, rank, rows, head_dim, C.byref(px), handle))
        return px, bytes(handle)

    def peer_exchange_attach(self, px: MfPeerExchange, peer: int, handle: bytes):
        buf = (C.c_uint8 * 64).from_buffer_copy(handle)
        self.check(lib.mf_peer_exchange_attach(self._h, C.byref(px), peer, buf))

    def peer_exchange_destroy(self, px: MfPeerExchange):
        self.check(lib.mf_peer_exchange_destroy(self._h, C.byref(px)))

    def paged_decode_push_merge(self, plan, cache, q, out, px: MfPeerExchange, step: int, pusher_mask: int, *, n_heads,
                                rope_positions=None, scale=None, k=None, v=None, cos=None, sin=None, rope=False,
                                rope_mode=ROPE_MODE_NEOX, append=False):
        """Sequence-sharded decode in one launch: partials pushed to every rank, merged by the same kernel."""
        scale = 1.0 / math.sqrt(cache.head_dim) if scale is None else scale
        a = MfPagedDecodeArgs(_ptr(q), _ptr(k), _ptr(v), None, _ptr(out), _ptr(cos), _ptr(sin), n_heads, int(rope),
                              rope_mode, int(append), scale)
        self.check(lib.mf_paged_decode_push_merge(self._h, plan._h, C.byref(cache), C.byref(a), _ptr(rope_positions),
                                                  C.byref(px), step, pusher_mask))

    def allgather_merge(self, comm, mine, gathered, rows, head_dim, out):
        """mf_allgather_merge: `mine` [rows*(head_dim+2)] f32, `gathered` [world, rows*(head_dim+2)] f32."""
        self.check(lib.mf_allgather_merge(self._h, comm, _ptr(mine), _ptr(gathered), gathered.shape[0], rows, head_dim, _ptr(out)))

    def set_allgather(self, fn):
        """fn: a ctypes callback ALLGATHER_FN (kept alive by the caller) or None."""
        self.check(lib.mf_context_set_allgather(self._h, C.cast(fn, vp) if fn is not None else None))

    def merge_pushed(self, px: MfPeerExchange, units_per_rank, step: int, rows: int, head_dim: int, out):
        arr = (u32 * 8)(*list(units_per_rank) + [0] * (8 - len(units_per_rank)))
        self.check(lib.mf_merge_pushed(self._h, C.byref(px), arr, step, rows, head_dim, _ptr(out)))

    def paged_prefill(self, cache: MfPagedKv, q, out, *, seq, q_len, kv_len, query_offset, n_heads, scale=None,
                      q_stride_h=None, q_stride_m=None, out_stride_h=None, out_stride_m=None):
        """Causal prefill attention over the pages of one sequence; q head-major [Hq, M, D] and out token-major
        [M, Hq*D] unless strides say otherwise."""
        d = cache.head_dim
        scale = 1.0 / math.sqrt(d) if scale is None else scale
        a = MfPagedPrefillArgs(_ptr(q), _ptr(out), seq, q_len, kv_len, query_offset, n_heads,
                               q_len * d if q_stride_h is None else q_stride_h, d if q_stride_m is None else q_stride_m,
                               d if out_stride_h is None else out_stride_h,
                               n_heads * d if out_stride_m is None else out_stride_m, scale)
        self.check(lib.mf_paged_prefill(self._h, C.byref(cache), C.byref(a)))

    def paged_copy_pages(self, cache: MfPagedKv, src_ids, dst_ids, n: int):
        """dst page <- src page for all kv heads of both pools; ids are device int32/uint32 tensors."""
        self.check(lib.mf_paged_copy_pages(self._h, C.byref(cache), _ptr(src_ids), _ptr(dst_ids), n))

    def paged_kv_append(self, cache: MfPagedKv, q, k, v, q_rot, cos, sin, *, n_heads, rope_mode=ROPE_MODE_NEOX,
                        apply_rope=True, seq=ALL_SEQUENCES, position_offset=0, seq_len=0):
        self.check(lib.mf_paged_kv_append(self._h, C.byref(cache), _ptr(q), _ptr(k), _ptr(v), _ptr(q_rot), _ptr(cos),
                                          _ptr(sin), n_heads, rope_mode, int(apply_rope), seq, position_offset,
                                          seq_len))

    @staticmethod
    def fused_qkv_args(x, w_q, w_k, w_v, *, k_dim, n_dim, n_kv, m, gamma=None, bias=None, out=None,
                       weights_per_block=0, epsilon=1e-6) -> MfFusedQkvArgs:
        """Arguments of FusedQkv (src/metals/gemv/qkv_step.rs:14-37); `bias` and `out` are (q, k, v) triples."""
        b = bias or (None, None, None)
        o = out or (None, None, None)
        a = MfFusedQkvArgs(_ptr(x), _ptr(w_q), _ptr(w_k), _ptr(w_v), _ptr(gamma), _ptr(b[0]), _ptr(b[1]), _ptr(b[2]),
                           _ptr(o[0]), _ptr(o[1]), _ptr(o[2]), k_dim, n_dim, n_kv, m, weights_per_block, epsilon)
        a._keep = (x, w_q, w_k, w_v, gamma, b, o)
        return a

    def fused_qkv(self, args: MfFusedQkvArgs):
        self.check(lib.mf_fused_qkv(self._h, C.byref(args)))

    def fused_qkv_kv_prep(self, args: MfFusedQkvArgs, q_rot, k_cache, v_cache, cos, sin,
                          params: KvPrepFusedParamsResolved):
        """FusedQkv and KvPrepFused in one launch."""
        ts = [tensor_arg(x) for x in (q_rot, k_cache, v_cache, cos, sin)]
        self.check(lib.mf_fused_qkv_kv_prep(self._h, C.byref(args), *[C.byref(t) for t in ts], C.byref(params)))

    def fused_qkv_paged_append(self, args: MfFusedQkvArgs, cache: MfPagedKv, q_rot, cos, sin, *, n_heads,
                               rope_mode=ROPE_MODE_NEOX, apply_rope=True, seq=ALL_SEQUENCES, position_offset=0):
        self.check(lib.mf_fused_qkv_paged_append(self._h, C.byref(args), C.byref(cache), _ptr(q_rot), _ptr(cos),
                                                 _ptr(sin), n_heads, rope_mode, int(apply_rope), seq, position_offset))

    def paged_gather(self, cache: MfPagedKv, use_v: bool, seq: int, length: int, out):
        self.check(lib.mf_paged_gather(self._h, C.byref(cache), int(use_v), seq, length, _ptr(out)))

    # -- 8-bit (FP8 E4M3) paged cache ------------------------------------------------------

    def paged_decode_kv8(self, plan: "DecodePlan", cache: "MfPagedKv8", q, out, *, n_heads, scale=None, k=None, v=None,
                         cos=None, sin=None, rope=False, rope_mode=ROPE_MODE_NEOX, append=False, q_rot=None):
        scale = 1.0 / math.sqrt(cache.head_dim) if scale is None else scale
        a = MfPagedDecodeArgs(_ptr(q), _ptr(k), _ptr(v), _ptr(q_rot), _ptr(out), _ptr(cos), _ptr(sin), n_heads,
                              int(rope), rope_mode, int(append), scale)
        self.check(lib.mf_paged_decode_kv8(self._h, plan._h, C.byref(cache), C.byref(a)))

    def paged_prefill_kv8(self, cache: "MfPagedKv8", q, out, workspace, *, seq, q_len, kv_len, query_offset, n_heads,
                          scale=None):
        """mf_paged_prefill_kv8: causal prefill over the 8-bit pages of one sequence; q head-major [Hq, M, D], out
        token-major [M, Hq*D]; `workspace`: a device tensor of at least paged_prefill_kv8_workspace_bytes bytes."""
        d = cache.head_dim
        scale = 1.0 / math.sqrt(d) if scale is None else scale
        a = MfPagedPrefillArgs(_ptr(q), _ptr(out), seq, q_len, kv_len, query_offset, n_heads, q_len * d, d, d, n_heads * d,
                               scale)
        self.check(lib.mf_paged_prefill_kv8(self._h, C.byref(cache), C.byref(a), _ptr(workspace),
                                            workspace.numel() * workspace.element_size()))

    def paged_decode_kv8_partial_push(self, plan: "DecodePlan", cache: "MfPagedKv8", q, px: MfPeerExchange, step: int, *,
                                      n_heads, rope_positions=None, scale=None, k=None, v=None, cos=None, sin=None,
                                      rope=False, rope_mode=ROPE_MODE_NEOX, append=False):
        scale = 1.0 / math.sqrt(cache.head_dim) if scale is None else scale
        a = MfPagedDecodeArgs(_ptr(q), _ptr(k), _ptr(v), None, None, _ptr(cos), _ptr(sin), n_heads, int(rope), rope_mode,
                              int(append), scale)
        self.check(lib.mf_paged_decode_kv8_partial_push(self._h, plan._h, C.byref(cache), C.byref(a), _ptr(rope_positions),
                                                        C.byref(px), step))

    def paged_decode_kv8_push_merge(self, plan: "DecodePlan", cache: "MfPagedKv8", q, out, px: MfPeerExchange, step: int,
                                    pusher_mask: int, *, n_heads, rope_positions=None, scale=None, k=None, v=None, cos=None,
                                    sin=None, rope=False, rope_mode=ROPE_MODE_NEOX, append=False):
        """mf_paged_decode_kv8_push_merge: the fused sequence-sharded step over the 8-bit cache."""
        scale = 1.0 / math.sqrt(cache.head_dim) if scale is None else scale
        a = MfPagedDecodeArgs(_ptr(q), _ptr(k), _ptr(v), None, _ptr(out), _ptr(cos), _ptr(sin), n_heads, int(rope),
                              rope_mode, int(append), scale)
        self.check(lib.mf_paged_decode_kv8_push_merge(self._h, plan._h, C.byref(cache), C.byref(a), _ptr(rope_positions),
                                                      C.byref(px), step, pusher_mask))

    def paged_decode_kv8_partial(self, plan: "DecodePlan", cache: "MfPagedKv8", q, rope_positions, acc, m, l, *, n_heads,
                                 scale=None, k=None, v=None, cos=None, sin=None, rope=False, rope_mode=ROPE_MODE_NEOX,
                                 append=False, q_rot=None):
        """mf_paged_decode_kv8_partial: a shard's unnormalised (acc, m, l) over the 8-bit cache."""
        scale = 1.0 / math.sqrt(cache.head_dim) if scale is None else scale
        a = MfPagedDecodeArgs(_ptr(q), _ptr(k), _ptr(v), _ptr(q_rot), None, _ptr(cos), _ptr(sin), n_heads,
                              int(rope), rope_mode, int(append), scale)
        self.check(lib.mf_paged_decode_kv8_partial(self._h, plan._h, C.byref(cache), C.byref(a), _ptr(rope_positions),
                                                   _ptr(acc), _ptr(m), _ptr(l)))

    def paged_kv8_append(self, cache: "MfPagedKv8", q, k, v, q_rot, cos, sin, *, n_heads, rope_mode=ROPE_MODE_NEOX,
                         apply_rope=True, seq=ALL_SEQUENCES, position_offset=0, seq_len=0):
        self.check(lib.mf_paged_kv8_append(self._h, C.byref(cache), _ptr(q), _ptr(k), _ptr(v), _ptr(q_rot), _ptr(cos),
                                           _ptr(sin), n_heads, rope_mode, int(apply_rope), seq, position_offset, seq_len))

    def paged_kv8_gather(self, cache: "MfPagedKv8", use_v: bool, seq: int, length: int, out):
        self.check(lib.mf_paged_kv8_gather(self._h, C.byref(cache), int(use_v), seq, length, _ptr(out)))


def paged_prefill_kv8_workspace_bytes(cache: "MfPagedKv8", kv_len: int) -> int:
    return int(lib.mf_paged_prefill_kv8_workspace_bytes(C.byref(cache), kv_len))


def flash_decode_static_scratch(stream, q, k, v, output, strides: MfFlashDecodeStrides, params: SdpaParams, n_heads,
                                batch=1):
    """mf_flash_decode_static_scratch: decode that allocates nothing (needs no Foundry).  `stream` is a raw
    cudaStream_t value (0 / None = the default stream)."""
    buf = C.create_string_buffer(256)
    st = lib.mf_flash_decode_static_scratch(None if not stream else int(stream), _ptr(q), _ptr(k), _ptr(v),
                                            _ptr(output), C.byref(strides), C.byref(params), n_heads, batch, buf, 256)
    if st != MF_OK:
        raise MetalError(st, buf.value.decode())


class PagePool:
    """Host-side page allocator with reference counts (mf_page_pool_*)."""

    def __init__(self, n_pages: int):
        h = vp()
        st = lib.mf_page_pool_create(n_pages, C.byref(h))
        if st != 0:
            raise MetalError(st, "mf_page_pool_create")
        self._h = h

    def close(self):
        if self._h:
            lib.mf_page_pool_destroy(self._h)
            self._h = None

    def _check(self, st, what):
        if st != 0:
            raise MetalError(st, what)

    def alloc(self, n: int) -> np.ndarray:
        ids = np.empty(n, np.uint32)
        self._check(lib.mf_page_pool_alloc(self._h, n, ids.ctypes.data_as(vp)), "page pool: not enough free pages")
        return ids

    def retain(self, ids):
        ids = np.ascontiguousarray(ids, np.uint32)
        self._check(lib.mf_page_pool_retain(self._h, ids.ctypes.data_as(vp), ids.size), "page pool: retain of a free page")

    def release(self, ids):
        ids = np.ascontiguousarray(ids, np.uint32)
        self._check(lib.mf_page_pool_release(self._h, ids.ctypes.data_as(vp), ids.size), "page pool: release of a free page")

    @property
    def free_count(self) -> int:
        return int(lib.mf_page_pool_free_count(self._h))

    def refcount(self, page: int) -> int:
        return int(lib.mf_page_pool_refcount(self._h, page))


class PrefixCache:
    """Prefix cache over shared pages (mf_prefix_cache_*); entry rules of src/model/executor.rs:1352-1636."""

    def __init__(self, pool: PagePool, page_size: int, max_entries: int | None = None):
        if max_entries is None:
            max_entries = int(lib.mf_prefix_cache_default_entries())
        h = vp()
        st = lib.mf_prefix_cache_create(pool._h, page_size, max_entries, C.byref(h))
        if st != 0:
            raise MetalError(st, "mf_prefix_cache_create")
        self._h, self.page_size, self.pool = h, page_size, pool

    def close(self):
        if self._h:
            lib.mf_prefix_cache_destroy(self._h)
            self._h = None

    def __len__(self):
        return int(lib.mf_prefix_cache_entries(self._h))

    def store(self, tokens, page_ids, key: str | None = None):
        tokens = np.ascontiguousarray(tokens, np.uint32)
        page_ids = np.ascontiguousarray(page_ids, np.uint32)
        st = lib.mf_prefix_cache_store(self._h, tokens.ctypes.data_as(vp), tokens.size,
                                       None if key is None else key.encode(), page_ids.ctypes.data_as(vp), page_ids.size)
        if st != 0:
            raise MetalError(st, "prefix cache store")

    def lookup(self, prompt, key: str | None = None):
        """Returns (matched tokens, page ids retained for the caller)."""
        prompt = np.ascontiguousarray(prompt, np.uint32)
        cap = (prompt.size + self.page_size - 1) // self.page_size + 1
        ids = np.empty(cap, np.uint32)
        matched, n = u32(0), u32(0)
        st = lib.mf_prefix_cache_lookup(self._h, prompt.ctypes.data_as(vp), prompt.size,
                                        None if key is None else key.encode(), C.byref(matched), ids.ctypes.data_as(vp), cap,
                                        C.byref(n))
        if st != 0:
            raise MetalError(st, "prefix cache lookup")
        return int(matched.value), ids[:n.value].copy()


class DecodePlan:
    """Equal-span work list of one batched decode step (see mf_decode_plan_create)."""

    def __init__(self, foundry: Foundry, kv_lens_host, n_heads, n_kv_heads, head_dim, page_size, max_ctas=0):
        import numpy as np

        self._f = foundry
        lens = np.ascontiguousarray(kv_lens_host, dtype=np.uint32)
        self.batch = int(lens.shape[0])
        h = vp()
        foundry.check(lib.mf_decode_plan_create(foundry._h, lens.ctypes.data, self.batch, n_heads, n_kv_heads, head_dim,
                                                page_size, max_ctas, C.byref(h)))
        self._h = h

    def update(self, kv_lens_host):
        import numpy as np

        lens = np.ascontiguousarray(kv_lens_host, dtype=np.uint32)
        assert lens.shape[0] == self.batch
        self._f.check(lib.mf_decode_plan_update(self._f._h, self._h, lens.ctypes.data))

    @property
    def ctas(self):
        return int(lib.mf_decode_plan_ctas(self._h))

    @property
    def cluster(self):
        return int(lib.mf_decode_plan_cluster(self._h))

    @property
    def items(self):
        return int(lib.mf_decode_plan_items(self._h))

    @property
    def tiles(self):
        return int(lib.mf_decode_plan_tiles(self._h))

    def close(self):
        if getattr(self, "_h", None) and getattr(self._f, "_h", None):
            lib.mf_decode_plan_destroy(self._f._h, self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def paged_kv(k_pool, v_pool, page_table, kv_lens, *, n_kv_heads, page_size, head_dim) -> MfPagedKv:
    """Describe torch-owned pools [n_pages, Hkv, P, D] and a [batch, stride] page table."""
    n_pages = k_pool.shape[0]
    desc = MfPagedKv(k_pool.data_ptr(), v_pool.data_ptr(), page_table.data_ptr(), kv_lens.data_ptr(), n_pages,
                     n_kv_heads, page_size, head_dim, page_table.shape[1], page_table.shape[0])
    desc._keep = (k_pool, v_pool, page_table, kv_lens)  # the descriptor holds raw pointers: keep their owners alive
    return desc


def kv8_v_pool_from_rows(rows):
    """Quantised V rows [n_pages, Hkv, P, 128] (numpy or torch, uint8) -> the V pool's byte order: dim-major blocks of
    16 keys inside each (page, kv head) run, [n_pages, Hkv, P/16, 128, 16], returned in the rows' shape."""
    n, h, p, d = rows.shape
    x = rows.reshape(n, h, p // 16, 16, d)
    x = x.transpose(0, 1, 2, 4, 3) if hasattr(x, "__array__") and not hasattr(x, "permute") else x.permute(0, 1, 2, 4, 3)
    return (x.copy() if not hasattr(x, "contiguous") else x.contiguous()).reshape(n, h, p, d)


def kv8_v_rows_from_pool(pool):
    """Inverse of kv8_v_pool_from_rows."""
    n, h, p, d = pool.shape
    x = pool.reshape(n, h, p // 16, d, 16)
    x = x.transpose(0, 1, 2, 4, 3) if hasattr(x, "__array__") and not hasattr(x, "permute") else x.permute(0, 1, 2, 4, 3)
    return (x.copy() if not hasattr(x, "contiguous") else x.contiguous()).reshape(n, h, p, d)


def paged_kv8(k_pool, v_pool, k_scales, v_scales, page_table, kv_lens, *, n_kv_heads, page_size) -> MfPagedKv8:
    """Describe torch-owned 8-bit pools (uint8; K [n_pages, Hkv, P, 128] row-major, V the same bytes per (page, kv head)
    in dim-major 16-key blocks, see kv8_v_pool_from_rows), their scale pools [n_pages, Hkv, P] (f32) and a
    [batch, stride] page table.  Page sizes 16, 32, 64."""
    desc = MfPagedKv8(k_pool.data_ptr(), v_pool.data_ptr(), k_scales.data_ptr(), v_scales.data_ptr(), page_table.data_ptr(),
                      kv_lens.data_ptr(), k_pool.shape[0], n_kv_heads, page_size, 128, page_table.shape[1], page_table.shape[0])
    desc._keep = (k_pool, v_pool, k_scales, v_scales, page_table, kv_lens)
    return desc


def rope_tables(rope_base: float, head_dim: int, n_pos: int, first_pos: int = 0, freq_factors=None):
    """Host RoPE cos/sin tables as numpy uint16 (f16 bits) arrays [n_pos, head_dim/2]."""
    import numpy as np

    half = head_dim // 2
    cos = np.empty((n_pos, half), np.uint16)
    sin = np.empty((n_pos, half), np.uint16)
    ff = None if freq_factors is None else np.ascontiguousarray(freq_factors, np.float32)
    st = lib.mf_rope_tables_host(rope_base, head_dim, first_pos, n_pos, None if ff is None else ff.ctypes.data,
                                 cos.ctypes.data, sin.ctypes.data)
    if st != MF_OK:
        raise MetalError(st, "mf_rope_tables_host")
    return cos, sin


def build_decode_plan_host(kv_lens, n_kv_heads: int, max_ctas: int):
    """Run the step planner on the host.  Returns (items [n, 8] uint32, cta_begin [n_ctas+1])."""
    import numpy as np

    lens = np.ascontiguousarray(kv_lens, dtype=np.uint32)
    cap = lens.shape[0] * n_kv_heads + max_ctas
    items = np.zeros((cap, 8), np.uint32)
    cta_begin = np.zeros(max_ctas + 1, np.uint32)
    n_ctas = u32(0)
    n = lib.mf_decode_plan_build_host(lens.ctypes.data, lens.shape[0], n_kv_heads, max_ctas, items.ctypes.data, cap,
                                      cta_begin.ctypes.data, C.byref(n_ctas))
    return items[:n].copy(), cta_begin[:n_ctas.value + 1].copy()


def build_decode_plan_host_clusters(kv_lens, n_kv_heads: int, max_ctas: int, max_cluster: int = 16, clusters_of_16: int = 0,
                                    clusters_of_8: int = 0):
    """The step planner for a launch that may take the cluster form.  Returns (items [n, 8] uint32, cluster size);
    cluster size 0: the plain form was chosen (items as build_decode_plan_host gives them)."""
    import numpy as np

    lens = np.ascontiguousarray(kv_lens, dtype=np.uint32)
    cap = lens.shape[0] * n_kv_heads + max_ctas
    items = np.zeros((cap, 8), np.uint32)
    n_ranges, cluster = u32(0), u32(0)
    n = lib.mf_decode_plan_build_host_clusters(lens.ctypes.data, lens.shape[0], n_kv_heads, max_ctas, max_cluster,
                                               clusters_of_16, clusters_of_8, items.ctypes.data, cap, C.byref(n_ranges),
                                               C.byref(cluster))
    return items[:n].copy(), int(cluster.value)


def align_capacity(n: int) -> int:
    return int(lib.mf_align_capacity(n))


def grown_capacity(current: int, required: int, max_context_len: int) -> int:
    return int(lib.mf_grown_capacity(current, required, max_context_len))


def prefill_split_k(kv_seq_len: int, q_seq_len: int) -> int:
    return int(lib.mf_prefill_split_k(kv_seq_len, q_seq_len))
