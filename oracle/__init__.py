"""ctypes binding of the CPU oracle (oracle/mf_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke entry and by the
bench's cpu-baseline / reference legs as the checker.  The product package never
imports this module.

`build()` compiles the C restatement with gcc into oracle/libmf_oracle.so;
`lib()` loads it (building on demand when gcc is available).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "libmf_oracle.so"
_SRC = _HERE / "mf_oracle.c"
_HDR = _HERE / "mf_oracle.h"
_LIB = None


def build(force: bool = False) -> Path:
    """Compile oracle/mf_oracle.c -> oracle/libmf_oracle.so (gcc, OpenMP)."""
    if not force and _SO.exists() and _SO.stat().st_mtime >= max(_SRC.stat().st_mtime, _HDR.stat().st_mtime):
        return _SO
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-fopenmp", "-std=c11",
           "-Wall", "-Wextra", "-o", str(_SO), str(_SRC), "-lm"]
    subprocess.run(cmd, check=True, cwd=_HERE)
    return _SO


u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
u32p = np.ctypeslib.ndpointer(dtype=np.uint32, flags="C_CONTIGUOUS")
f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
f64p = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")
u32 = C.c_uint32
u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")

_FAST_SRC = _HERE / "mf_oracle_fast.c"
_FAST_LIB = None


def _cpu_tag() -> str:
    """A short tag of this machine's CPU features: the fast build uses -march=native, so a library
    built on one machine must not be loaded on another."""
    import hashlib

    flags = ""
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("flags"):
                flags = line
                break
    except OSError:
        pass
    return hashlib.sha1(flags.encode()).hexdigest()[:10]


def build_fast(force: bool = False) -> Path:
    """Compile oracle/mf_oracle_fast.c for THIS machine (gcc -O3 -march=native, OpenMP) ->
    oracle/libmf_oracle_fast.<cpu tag>.so."""
    so = _HERE / f"libmf_oracle_fast.{_cpu_tag()}.so"
    if not force and so.exists() and so.stat().st_mtime >= _FAST_SRC.stat().st_mtime:
        return so
    cmd = ["gcc", "-O3", "-march=native", "-fPIC", "-shared", "-fopenmp", "-std=c11", "-Wall", "-Wextra", "-o", str(so),
           str(_FAST_SRC), "-lm"]
    subprocess.run(cmd, check=True, cwd=_HERE)
    return so


def fast_lib() -> C.CDLL:
    """The timed CPU arm (see mf_oracle_fast.c).  Built on first use on the machine that runs it."""
    global _FAST_LIB
    if _FAST_LIB is not None:
        return _FAST_LIB
    L = C.CDLL(str(build_fast()))
    L.mfo_fast_paged_decode_layer.argtypes = [u16p, u16p, u16p, u16p, u16p, u16p, u16p, u32p, u32, u32p, u32, u32, u32, u32,
                                              u32, u32, C.c_float, u16p]
    L.mfo_fast_paged_decode_layer.restype = C.c_int
    L.mfo_fast_num_threads.restype = C.c_int
    L.mfo_fast_set_num_threads.argtypes = [C.c_int]
    L.mfo_fast_simd.restype = C.c_int
    _FAST_LIB = L
    return L


class KvPrepParams(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "d_model", "kv_dim", "head_dim", "n_heads", "n_kv_heads", "group_size", "seq_len",
        "position_offset", "max_seq_len", "total_elements", "rope_mode", "layer_idx",
        "no_rope_layer_step")]


def lib() -> C.CDLL:
    global _LIB
    if _LIB is not None:
        return _LIB
    try:
        build()
    except (OSError, subprocess.CalledProcessError):
        if not _SO.exists():
            raise
    L = C.CDLL(str(_SO))
    L.mfo_f32_to_f16.argtypes = [C.c_float]
    L.mfo_f32_to_f16.restype = C.c_uint16
    L.mfo_f16_to_f32.argtypes = [C.c_uint16]
    L.mfo_f16_to_f32.restype = C.c_float
    L.mfo_lcg_fill_f16.argtypes = [u32, u16p, C.c_size_t, C.c_float]
    L.mfo_lcg_fill_f16.restype = u32
    L.mfo_splitmix64.argtypes = [C.c_uint64]
    L.mfo_splitmix64.restype = C.c_uint64
    L.mfo_normal_fill_f16.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64, u16p, C.c_size_t]
    L.mfo_rope_tables.argtypes = [C.c_float, u32, u32, u32, C.c_void_p, u16p, u16p]
    L.mfo_rope_neox.argtypes = [u16p, u16p, u16p, u16p, u32, u32, u32, C.c_size_t]
    L.mfo_kv_rearrange.argtypes = [u16p, u16p, u32, u32, u32, u32, u32, u32]
    L.mfo_kv_cache_write.argtypes = [u16p, u16p, u32, u32, u32, u32, u32]
    L.mfo_kv_cache_write_repeat.argtypes = [u16p, u16p, u32, u32, u32, u32, u32, u32]
    L.mfo_kv_cache_read.argtypes = [u16p, u16p, u32, u32, u32, u32]
    L.mfo_repeat_kv_heads.argtypes = [u16p, u16p, u32, u32, u32, u32]
    L.mfo_kv_cache_grow.argtypes = [u16p, u16p, u32, u32, u32, u32, u32]
    L.mfo_paged_scatter.argtypes = [u16p, u16p, u32p, u32, u32, u32, u32, u32]
    L.mfo_kv_prep_fused.argtypes = [u16p, u16p, u16p, u16p, u16p, u16p, u16p, u16p,
                                    C.POINTER(KvPrepParams), C.c_int]
    L.mfo_fused_qkv.argtypes = [u16p, u16p, u16p, u16p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, u32, u32, u32,
                                u32, u32, C.c_float, u16p, u16p, u16p]
    L.mfo_paged_kv_append.argtypes = [u16p, u16p, u16p, u16p, u16p, u16p, u16p, u16p, u32p, u32,
                                      u32p, u32, u32, u32, u32, u32, u32, C.c_int]
    L.mfo_paged_gather.argtypes = [u16p, u32p, u32, u32, u32, u32, u16p]
    L.mfo_decode_online.argtypes = [u16p, u16p, u16p, u32, u32, u32, u32, u32, u32, C.c_float,
                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.mfo_decode_blocked.argtypes = [u16p, u16p, u16p, u32, u32, u32, u32, u32, u32, C.c_float, u16p]
    L.mfo_decode_gold.argtypes = [u16p, u16p, u16p, u32, u32, u32, u32, u32, C.c_float, f64p]
    L.mfo_cpu_sdpa_attention.argtypes = [u16p, u16p, u16p, u16p, u16p, u32, u32, u32, u16p]
    L.mfo_prefill_causal.argtypes = [u16p, u16p, u16p, u32, u32, u32, u32, u32, u32, u32,
                                     C.c_float, u32, u32, C.c_void_p, C.c_void_p, C.c_void_p,
                                     C.c_void_p]
    L.mfo_prefill_gold.argtypes = [u16p, u16p, u16p, u32, u32, u32, u32, u32, u32, u32, C.c_float,
                                   f64p]
    L.mfo_splitk_tile_range.argtypes = [u32, u32, u32, C.POINTER(u32), C.POINTER(u32)]
    L.mfo_merge_partials.argtypes = [f32p, f32p, f32p, u32, u32, u32, u16p]
    L.mfo_e4m3_to_f32.argtypes = [C.c_uint8]
    L.mfo_e4m3_to_f32.restype = C.c_float
    L.mfo_f32_to_e4m3.argtypes = [C.c_float]
    L.mfo_f32_to_e4m3.restype = C.c_uint8
    L.mfo_quantize_row_e4m3.argtypes = [u16p, u32, u8p, C.POINTER(C.c_float)]
    L.mfo_kv8_v_index.argtypes = [C.c_size_t, u32, u32, u32]
    L.mfo_kv8_v_index.restype = C.c_size_t
    L.mfo_paged_kv8_append.argtypes = [u16p, u16p, u16p, u16p, u8p, u8p, f32p, f32p, u16p, u16p, u32p, u32, u32p, u32, u32,
                                       u32, u32, u32, u32, C.c_int]
    L.mfo_decode_kv8.argtypes = [u16p, u8p, u8p, f32p, f32p, u32p, u32, u32, u32, u32, u32, C.c_float, u16p, C.c_void_p]
    L.mfo_sdpa_materialized.argtypes = [u16p, u16p, u16p, u32, u32, u32, u32, u32, u32, C.c_uint64, C.c_uint64,
                                        C.c_uint64, C.c_uint64, C.c_int, u32, C.c_float, u16p]
    L.mfo_paged_decode_layer.argtypes = [u16p, u16p, u16p, u16p, u16p, u16p, u16p, u32p, u32, u32p,
                                         u32, u32, u32, u32, u32, u32, C.c_float, u16p]
    L.mfo_num_threads.restype = C.c_int
    L.mfo_set_num_threads.argtypes = [C.c_int]
    _LIB = L
    return L


# ----------------------------------------------------------------- helpers ---

def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def f16_bits(x: np.ndarray) -> np.ndarray:
    """float16 array -> uint16 view (C-contiguous)."""
    return np.ascontiguousarray(x).view(np.uint16)


def lcg_fill(state: int, n: int, scale: float):
    out = np.empty(n, np.uint16)
    state = lib().mfo_lcg_fill_f16(state, out, n, scale)
    return out, state


def normal_fill(seed: int, tensor_id: int, n: int, first: int = 0) -> np.ndarray:
    out = np.empty(n, np.uint16)
    lib().mfo_normal_fill_f16(seed, tensor_id, first, out, n)
    return out


def rope_tables(theta: float, head_dim: int, n_pos: int, first_pos: int = 0, freq_factors=None):
    half = head_dim // 2
    cos = np.empty((n_pos, half), np.uint16)
    sin = np.empty((n_pos, half), np.uint16)
    ff = None
    if freq_factors is not None:
        ff = np.ascontiguousarray(freq_factors, np.float32)
    lib().mfo_rope_tables(theta, head_dim, first_pos, n_pos, _ptr(ff), cos, sin)
    return cos, sin


def kv_prep_fused(q, k, v, k_cache, v_cache, cos, sin, *, n_heads, n_kv_heads, head_dim, seq_len,
                  position_offset, max_seq_len, rope_mode, layer_idx=0, no_rope_layer_step=0,
                  expanded=False):
    """Returns q_rot; k_cache / v_cache are updated in place."""
    p = KvPrepParams(n_heads * head_dim, n_kv_heads * head_dim, head_dim, n_heads, n_kv_heads,
                     n_heads // n_kv_heads, seq_len, position_offset, max_seq_len,
                     n_heads * seq_len * head_dim, rope_mode, layer_idx, no_rope_layer_step)
    q_rot = np.empty(n_heads * seq_len * head_dim, np.uint16)
    lib().mfo_kv_prep_fused(q, k, v, q_rot, k_cache, v_cache, cos, sin, C.byref(p), int(expanded))
    return q_rot


def fused_qkv(x, w_q, w_k, w_v, *, m, k_dim, n_dim, n_kv, gamma=None, b_q=None, b_k=None, b_v=None,
              weights_per_block=0, eps=1e-6):
    """RMSNorm -> Q/K/V projection (+bias) as the reference's FusedQkv computes it
    (src/metals/gemv/qkv_project.metal:4-272).  All arrays are f16 bit patterns (uint16)."""
    q = np.empty(m * n_dim, np.uint16)
    k = np.empty(m * n_kv, np.uint16)
    v = np.empty(m * n_kv, np.uint16)
    lib().mfo_fused_qkv(x, w_q, w_k, w_v, _ptr(gamma), _ptr(b_q), _ptr(b_k), _ptr(b_v), m, k_dim, n_dim, n_kv,
                        weights_per_block, eps, q, k, v)
    return q, k, v


def decode_online(q_rot, k_cache, v_cache, *, n_heads, cache_heads, head_dim, capacity, kv_len,
                  scale, key_begin=0, partials=False):
    out = np.empty(n_heads * head_dim, np.uint16)
    acc = m = l = None
    if partials:
        acc = np.empty((n_heads, head_dim), np.float32)
        m = np.empty(n_heads, np.float32)
        l = np.empty(n_heads, np.float32)
    lib().mfo_decode_online(q_rot, k_cache, v_cache, n_heads, cache_heads, head_dim, capacity,
                            key_begin, kv_len, scale, _ptr(out), _ptr(acc), _ptr(m), _ptr(l))
    return (out, acc, m, l) if partials else out


def decode_blocked(q_rot, k_cache, v_cache, *, n_heads, cache_heads, head_dim, capacity, kv_len,
                   scale, block_keys):
    out = np.zeros(n_heads * head_dim, np.uint16)
    lib().mfo_decode_blocked(q_rot, k_cache, v_cache, n_heads, cache_heads, head_dim, capacity,
                             kv_len, block_keys, scale, out)
    return out


def decode_gold(q_rot, k_cache, v_cache, *, n_heads, cache_heads, head_dim, capacity, kv_len, scale):
    out = np.empty((n_heads, head_dim), np.float64)
    lib().mfo_decode_gold(q_rot, k_cache, v_cache, n_heads, cache_heads, head_dim, capacity, kv_len,
                          scale, out)
    return out


def prefill_causal(q, k_cache, v_cache, *, n_heads, cache_heads, head_dim, capacity, q_len, kv_len,
                   query_offset, scale, tile_begin=0, tile_end=None, partials=False):
    if tile_end is None:
        tile_end = (kv_len + 31) // 32
    out = np.empty((q_len, n_heads * head_dim), np.uint16)
    acc = m = l = None
    if partials:
        acc = np.empty((n_heads, q_len, head_dim), np.float32)
        m = np.empty((n_heads, q_len), np.float32)
        l = np.empty((n_heads, q_len), np.float32)
    lib().mfo_prefill_causal(q, k_cache, v_cache, n_heads, cache_heads, head_dim, capacity, q_len,
                             kv_len, query_offset, scale, tile_begin, tile_end, _ptr(out),
                             _ptr(acc), _ptr(m), _ptr(l))
    return (out, acc, m, l) if partials else out


def prefill_gold(q, k_cache, v_cache, *, n_heads, cache_heads, head_dim, capacity, q_len, kv_len,
                 query_offset, scale):
    out = np.empty((q_len, n_heads * head_dim), np.float64)
    lib().mfo_prefill_gold(q, k_cache, v_cache, n_heads, cache_heads, head_dim, capacity, q_len,
                           kv_len, query_offset, scale, out)
    return out


def sdpa_materialized(q, k, v, *, n_heads, head_dim, m, kv_len, causal, query_offset, scale, q_head_major,
                      k_rows=None):
    """The reference's materialised fallback (S and P stored as f16).  q is token-major [m, H*D]
    or, with q_head_major, packed head-major [H, m, D]; k, v are [H, k_rows, D]; returns the
    token-major output [m, H*D] as f16 bits."""
    k_rows = kv_len if k_rows is None else k_rows
    D = head_dim
    out = np.zeros((m, n_heads * D), np.uint16)
    qs_h, qs_m = (m * D, D) if q_head_major else (D, n_heads * D)
    lib().mfo_sdpa_materialized(np.ascontiguousarray(q).ravel(), np.ascontiguousarray(k).ravel(),
                                np.ascontiguousarray(v).ravel(), n_heads, D, m, kv_len, k_rows, k_rows, qs_h, qs_m,
                                D, n_heads * D, int(bool(causal)), query_offset, scale, out.reshape(-1))
    return out


def merge_partials(acc, m, l):
    """acc [S, rows, D] f32, m/l [S, rows] f32 -> [rows, D] f16 bits."""
    acc = np.ascontiguousarray(acc, np.float32)
    m = np.ascontiguousarray(m, np.float32)
    l = np.ascontiguousarray(l, np.float32)
    S, rows, D = acc.shape
    out = np.empty((rows, D), np.uint16)
    lib().mfo_merge_partials(acc, m, l, S, rows, D, out)
    return out


def h2f(bits: np.ndarray) -> np.ndarray:
    return np.asarray(bits, np.uint16).view(np.float16).astype(np.float32)
