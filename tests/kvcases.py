"""Shared case builders for the parity tests: seeded inputs (host, via the oracle's
generators), device upload helpers and f16 comparison utilities."""
from __future__ import annotations

import numpy as np

import oracle

SEED = 0x5EED


# ------------------------------------------------------------------ f16 utils ---

def ordered(bits: np.ndarray) -> np.ndarray:
    """Map f16 bit patterns to integers whose difference is the ulp distance."""
    b = bits.astype(np.int32)
    return np.where(b & 0x8000, -(b & 0x7FFF), b)


def ulp_distance(a_bits: np.ndarray, b_bits: np.ndarray) -> int:
    return int(np.max(np.abs(ordered(a_bits.ravel()) - ordered(b_bits.ravel())))) if a_bits.size else 0


def max_abs(a_bits: np.ndarray, ref) -> float:
    a = oracle.h2f(a_bits).astype(np.float64).ravel()
    r = (oracle.h2f(ref) if ref.dtype == np.uint16 else ref).astype(np.float64).ravel()
    return float(np.max(np.abs(a - r))) if a.size else 0.0


def dev(bits: np.ndarray):
    """uint16 f16-bit array -> torch.float16 CUDA tensor of the same shape."""
    import torch

    return torch.from_numpy(np.ascontiguousarray(bits).view(np.float16)).cuda()


def dev_u32(a: np.ndarray):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.uint32).view(np.int32)).cuda()


def host(t) -> np.ndarray:
    """torch.float16 tensor -> uint16 bits (numpy)."""
    return t.detach().cpu().contiguous().numpy().view(np.uint16)


# ------------------------------------------------------------------- inputs ---

def normal(tensor_id: int, n: int, seed: int = SEED) -> np.ndarray:
    return oracle.normal_fill(seed, tensor_id, n)


def lcg(seed: int, n: int, scale: float) -> np.ndarray:
    out, _ = oracle.lcg_fill(seed, n, scale)
    return out


class ContigCase:
    """One layer of the contiguous cache path: `cached` rows already in the cache,
    M new tokens appended at position `cached`, then attention over cached+M keys."""

    def __init__(self, *, n_heads, n_kv_heads, head_dim, cached, m=1, capacity=None, theta=1e6, rope_mode=0,
                 seed=SEED, gen="normal", scale=1.0, expanded=False, poison=False):
        self.Hq, self.Hkv, self.D, self.M = n_heads, n_kv_heads, head_dim, m
        self.cached, self.L = cached, cached + m
        self.cap = capacity if capacity is not None else max(self.L, 1)
        self.rope_mode, self.expanded = rope_mode, expanded
        self.cache_heads = n_heads if expanded else n_kv_heads
        self.G = n_heads // n_kv_heads
        D = head_dim
        if gen == "normal":
            g = lambda tid, n: normal(tid, n, seed)
        else:
            st = [seed]

            def g(tid, n):
                out, st[0] = oracle.lcg_fill(st[0], n, scale)
                return out
        self.q = g(1, m * n_heads * D).reshape(m, n_heads * D)
        self.k = g(2, m * n_kv_heads * D).reshape(m, n_kv_heads * D)
        self.v = g(3, m * n_kv_heads * D).reshape(m, n_kv_heads * D)
        # Cache rows [0, cached) hold N(0,1) values ("already roped" keys); rows past that
        # are zero, or NaN patterns when `poison` asks for proof that they are never used.
        fill = 0x7E00 if poison else 0
        self.k_cache = np.full((self.cache_heads, self.cap, D), fill, np.uint16)
        self.v_cache = np.full((self.cache_heads, self.cap, D), fill, np.uint16)
        kc = g(4, n_kv_heads * cached * D).reshape(n_kv_heads, cached, D)
        vc = g(5, n_kv_heads * cached * D).reshape(n_kv_heads, cached, D)
        rep = self.G if expanded else 1
        self.k_cache[:, :cached] = np.repeat(kc, rep, axis=0)
        self.v_cache[:, :cached] = np.repeat(vc, rep, axis=0)
        self.cos, self.sin = oracle.rope_tables(theta, D, self.cap)
        self.scale = np.float32(1.0) / np.sqrt(np.float32(D))

    def oracle_append(self, layer_idx=0, no_rope_layer_step=0):
        """Returns (q_rot [Hq*M*D], k_cache', v_cache') from the oracle."""
        kc, vc = self.k_cache.copy(), self.v_cache.copy()
        q_rot = oracle.kv_prep_fused(self.q, self.k, self.v, kc, vc, self.cos, self.sin, n_heads=self.Hq,
                                     n_kv_heads=self.Hkv, head_dim=self.D, seq_len=self.M,
                                     position_offset=self.cached, max_seq_len=self.cap, rope_mode=self.rope_mode,
                                     layer_idx=layer_idx, no_rope_layer_step=no_rope_layer_step,
                                     expanded=self.expanded)
        return q_rot, kc, vc


class PagedCase:
    """Batched paged decode: sequence b has `cached[b]` tokens in the pool, one new
    token is appended at position cached[b]; pages are a seeded permutation of the pool."""

    def __init__(self, *, batch, n_heads, n_kv_heads, head_dim, page_size, cached, theta=1e6, rope_mode=0,
                 seed=SEED, extra_pages=3, poison=True):
        self.B, self.Hq, self.Hkv, self.D, self.P = batch, n_heads, n_kv_heads, head_dim, page_size
        self.rope_mode = rope_mode
        self.cached = np.asarray(cached, np.uint32)
        self.kv_lens = self.cached + 1
        D, P = head_dim, page_size
        pages_per_seq = (self.kv_lens + P - 1) // P
        self.n_pages = int(pages_per_seq.sum()) + extra_pages
        rng = np.random.default_rng(seed)
        perm = rng.permutation(self.n_pages).astype(np.uint32)
        self.pt_stride = int(pages_per_seq.max())
        # Unused table entries point past the pool on purpose: they must never be read.
        self.page_table = np.full((batch, self.pt_stride), 0x7FFFFFF0, np.uint32)
        o = 0
        for b in range(batch):
            n = int(pages_per_seq[b])
            self.page_table[b, :n] = perm[o:o + n]
            o += n
        fill = 0x7E00 if poison else 0
        self.k_pool = np.full((self.n_pages, n_kv_heads, P, D), fill, np.uint16)
        self.v_pool = np.full((self.n_pages, n_kv_heads, P, D), fill, np.uint16)
        for b in range(batch):
            c = int(self.cached[b])
            kc = normal(100 + 2 * b, n_kv_heads * c * D, seed).reshape(n_kv_heads, c, D)
            vc = normal(101 + 2 * b, n_kv_heads * c * D, seed).reshape(n_kv_heads, c, D)
            for t0 in range(0, c, P):
                n = min(P, c - t0)
                page = self.page_table[b, t0 // P]
                self.k_pool[page, :, :n] = kc[:, t0:t0 + n]
                self.v_pool[page, :, :n] = vc[:, t0:t0 + n]
        self.q = normal(1, batch * n_heads * D, seed).reshape(batch, n_heads * D)
        self.k = normal(2, batch * n_kv_heads * D, seed).reshape(batch, n_kv_heads * D)
        self.v = normal(3, batch * n_kv_heads * D, seed).reshape(batch, n_kv_heads * D)
        max_pos = int(self.kv_lens.max())
        self.cos, self.sin = oracle.rope_tables(theta, D, max_pos)
        self.scale = np.float32(1.0) / np.sqrt(np.float32(D))

    def oracle_step(self):
        """Append + attend with the oracle.  Returns (q_rot, k_pool', v_pool', out [B, Hq*D], gold f64)."""
        L = oracle.lib()
        kp, vp = self.k_pool.copy(), self.v_pool.copy()
        q_rot = np.empty_like(self.q)
        L.mfo_paged_kv_append(self.q, self.k, self.v, q_rot, kp, vp, self.cos, self.sin, self.page_table,
                              self.pt_stride, self.cached, self.B, self.Hq, self.Hkv, self.D, self.P,
                              self.rope_mode, 1)
        out = np.empty((self.B, self.Hq * self.D), np.uint16)
        gold = np.empty((self.B, self.Hq, self.D), np.float64)
        for b in range(self.B):
            n = int(self.kv_lens[b])
            kc = np.empty((self.Hkv, n, self.D), np.uint16)
            vc = np.empty((self.Hkv, n, self.D), np.uint16)
            L.mfo_paged_gather(kp, self.page_table[b], n, self.Hkv, self.P, self.D, kc)
            L.mfo_paged_gather(vp, self.page_table[b], n, self.Hkv, self.P, self.D, vc)
            out[b] = oracle.decode_online(q_rot[b], kc, vc, n_heads=self.Hq, cache_heads=self.Hkv, head_dim=self.D,
                                          capacity=n, kv_len=n, scale=self.scale)
            gold[b] = oracle.decode_gold(q_rot[b], kc, vc, n_heads=self.Hq, cache_heads=self.Hkv, head_dim=self.D,
                                         capacity=n, kv_len=n, scale=self.scale)
        return q_rot, kp, vp, out, gold
