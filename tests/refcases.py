"""The fixtures of the reference's own attention parity tests, restated: same LCG seeds, draw order,
scales and shapes (paths relative to crates/metallic-foundry/ of the reference).  The reference stores
no outputs; what it asserts on these inputs is a bound between its flash kernels and its materialised
path, and these cases let the same assertion be replayed here."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

import oracle

DECODE_TOL = 6e-2   # tests/flashattention_decode_parity.rs:190
PREFILL_TOL = 8e-2  # tests/flashattention_prefill_parity.rs:136-139


@dataclass
class RefCase:
    name: str
    n_heads: int
    head_dim: int
    m: int
    kv_len: int
    capacity: int
    query_offset: int
    q: np.ndarray          # token-major [m, H*D] unless q_head_major
    k: np.ndarray          # [H, capacity, D] (expanded cache: one K/V head per query head)
    v: np.ndarray
    q_head_major: bool = False  # contents packed [H, m, D]
    m_cap: int = 0              # > 0: the bound tensor is [1, m_cap, H*D] / output [m_cap, H*D]
    split_k: int = 1

    @property
    def scale(self):
        return np.float32(1.0) / np.sqrt(np.float32(self.head_dim))


def _draw(seed, n_heads, head_dim, m, capacity, scale):
    st = seed & 0xFFFFFFFF
    q, st = oracle.lcg_fill(st, m * n_heads * head_dim, scale)
    k, st = oracle.lcg_fill(st, n_heads * capacity * head_dim, scale)
    v, st = oracle.lcg_fill(st, n_heads * capacity * head_dim, scale)
    return q, k.reshape(n_heads, capacity, head_dim), v.reshape(n_heads, capacity, head_dim)


def decode_cases():
    """tests/flashattention_decode_parity.rs:117-346."""
    out = []
    for name, h, d, kv, cap, seed, sc in [("small", 14, 64, 128, 128, 1, 0.25), ("odd_kv_len", 14, 64, 27, 64, 7, 0.25),
                                          ("d128", 8, 128, 128, 128, 42, 0.1)]:
        q, k, v = _draw(seed, h, d, 1, cap, sc)
        out.append(RefCase(name, h, d, 1, kv, cap, kv - 1, q.reshape(1, h * d), k, v))
    return out


def _prefill_case(h, d, m, kv_len, query_offset, split_k=1):
    """run_prefill_case (tests/flashattention_prefill_parity.rs:75-141)."""
    seed = 123 ^ (((m * 31) & 0xFFFFFFFF) ^ ((kv_len * 131) & 0xFFFFFFFF))
    q, k, v = _draw(seed, h, d, m, kv_len, 0.25)
    return RefCase(f"h{h}_d{d}_m{m}_kv{kv_len}_sk{split_k}", h, d, m, kv_len, kv_len, query_offset, q.reshape(m, h * d), k,
                   v, split_k=split_k)


def prefill_cases():
    """tests/flashattention_prefill_parity.rs:143-538."""
    out = []
    for h, d in ((14, 64), (8, 128)):
        for m in (7, 16, 17):                                   # :143-163 (WARPS=4 tiles)
            out.append(_prefill_case(h, d, m, m, 0))
        for m, kv, off in ((32, 256, 224), (17, 256, 239), (32, 1024, 992)):  # :165-186, split-K forced to 4
            out.append(_prefill_case(h, d, m, kv, off, split_k=4))
    for m in (1, 2, 7, 17, 31, 32, 33):                         # :507-522
        out.append(_prefill_case(14, 64, m, m, 0))
        out.append(_prefill_case(14, 64, m, m + 64, 64))
    for m in (1, 2, 17, 31, 32, 33):                            # :524-538
        out.append(_prefill_case(8, 128, m, m, 0))
        out.append(_prefill_case(8, 128, m, m + 64, 64))
    # the four tests that draw with fixed seeds (:188-505)
    for name, seed, m, kv in (("no_prefix", 11, 32, 32), ("with_prefix", 19, 32, 96), ("partial_tile", 29, 26, 26)):
        q, k, v = _draw(seed, 14, 64, m, kv, 0.25)
        out.append(RefCase(name, 14, 64, m, kv, kv, kv - m, q.reshape(m, 14 * 64), k, v))
    # Q bound as [1, M_cap, d_model] whose contents are head-major packed over the true M (:383-505)
    m, m_cap, h, d = 26, 32, 14, 64
    st = 41
    packed, st = oracle.lcg_fill(st, h * m * d, 0.25)
    k, st = oracle.lcg_fill(st, h * m * d, 0.25)
    v, st = oracle.lcg_fill(st, h * m * d, 0.25)
    out.append(RefCase("q_token_meta_head_major_contents", h, d, m, m, m, 0, packed.reshape(h, m, d), k.reshape(h, m, d),
                       v.reshape(h, m, d), q_head_major=True, m_cap=m_cap))
    return out


def materialized(case: RefCase) -> np.ndarray:
    """What the reference compares its flash kernels with: token-major [m, H*D] f16 bits."""
    return oracle.sdpa_materialized(case.q, case.k, case.v, n_heads=case.n_heads, head_dim=case.head_dim, m=case.m,
                                    kv_len=case.kv_len, causal=True, query_offset=case.query_offset, scale=case.scale,
                                    q_head_major=case.q_head_major, k_rows=case.capacity)


def q_head_major(case: RefCase) -> np.ndarray:
    """Q as packed head-major [H, m, D] bits (the layout the flash oracle functions take)."""
    if case.q_head_major:
        return np.ascontiguousarray(case.q)
    return np.ascontiguousarray(case.q.reshape(case.m, case.n_heads, case.head_dim).transpose(1, 0, 2))


def misaligned_case():
    """tests/sdpa_head_stride_misaligned.rs:9-112: closed-form inputs (no RNG) and the test's own
    CPU function (two-pass f32 softmax over the unrounded f32 inputs).  Returns q [H, m, D],
    k, v [H, seq_k, D] as f16 bits and the expected token-major [m, H*D] f32 output."""
    n_heads, head_dim, m, seq_k = 2, 64, 17, 15
    h = np.arange(n_heads, dtype=np.float32)[:, None, None] + np.float32(1)
    t = np.arange(m, dtype=np.float32)[None, :, None] + np.float32(1)
    s = np.arange(seq_k, dtype=np.float32)[None, :, None] + np.float32(1)
    d = np.arange(head_dim, dtype=np.float32)[None, None, :]
    q32 = (h * t * (d + np.float32(1)) * np.float32(0.001)).astype(np.float32)
    k32 = (h * s * (d + np.float32(1)) * np.float32(0.00001)).astype(np.float32)
    v32 = (h * s * ((d % 7) + np.float32(1)) * np.float32(0.0001)).astype(np.float32)
    scale = np.float32(1.0) / np.sqrt(np.float32(head_dim))
    expected = np.zeros((m, n_heads * head_dim), np.float32)
    for ti in range(m):
        for hi in range(n_heads):
            scores = np.zeros(seq_k, np.float32)
            for si in range(seq_k):
                dot = np.float32(0)
                for di in range(head_dim):
                    dot = np.float32(dot + q32[hi, ti, di] * k32[hi, si, di])
                scores[si] = dot * scale
            e = np.exp((scores - scores.max()).astype(np.float32)).astype(np.float32)
            total = np.float32(0)
            for x in e:
                total = np.float32(total + x)
            for si in range(seq_k):
                expected[ti, hi * head_dim:(hi + 1) * head_dim] += np.float32(e[si] / total) * v32[hi, si]
    bits = lambda a: np.ascontiguousarray(a.astype(np.float16)).view(np.uint16)
    return dict(n_heads=n_heads, head_dim=head_dim, m=m, seq_k=seq_k, q=bits(q32), k=bits(k32), v=bits(v32), scale=scale,
                expected=expected)


def materialized_m4_case(seed=123):
    """tests/sdpa_materialized_prefill_parity.rs:10-116 (m=4, L=8, H=2, D=64, non-causal).  The test
    draws uniform(-0.5, 0.5) from Rust's StdRng, whose stream is not reproduced here: the same
    distribution from a seeded numpy generator stands in; the CPU function is the test's."""
    n_heads, head_dim, m, kv = 2, 64, 4, 8
    rng = np.random.default_rng(seed)
    q32 = rng.uniform(-0.5, 0.5, (n_heads, m, head_dim)).astype(np.float16)
    k32 = rng.uniform(-0.5, 0.5, (n_heads, kv, head_dim)).astype(np.float16)
    v32 = rng.uniform(-0.5, 0.5, (n_heads, kv, head_dim)).astype(np.float16)
    scale = np.float32(1.0) / np.sqrt(np.float32(head_dim))
    qf, kf, vf = q32.astype(np.float32), k32.astype(np.float32), v32.astype(np.float32)
    expected = np.zeros((m, n_heads * head_dim), np.float32)
    for h in range(n_heads):
        scores = (qf[h] @ kf[h].T).astype(np.float32) * scale
        e = np.exp(scores - scores.max(axis=1, keepdims=True)).astype(np.float32)
        p = e / e.sum(axis=1, keepdims=True)
        expected[:, h * head_dim:(h + 1) * head_dim] = p @ vf[h]
    return dict(n_heads=n_heads, head_dim=head_dim, m=m, seq_k=kv, q=q32.view(np.uint16), k=k32.view(np.uint16),
                v=v32.view(np.uint16), scale=scale, expected=expected)
