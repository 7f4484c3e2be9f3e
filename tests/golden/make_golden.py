"""Regenerate tests/golden/kv_path_golden.npz from the CPU oracle.

    python tests/golden/make_golden.py

The reference stores no expected outputs for this path and cannot run here (Rust + Metal), so
these vectors are outputs of the oracle (oracle/mf_oracle.c) on the reference's own test shapes
with its deterministic LCG inputs (tests/flashattention_decode_parity.rs:15-30 of the reference).
They pin the oracle against regressions and give the GPU tests a fixed target; they are not
outputs of the reference itself.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import oracle  # noqa: E402
from kvcases import ContigCase  # noqa: E402

# (name, n_heads, n_kv_heads, head_dim, cached, m, capacity, rope_mode, lcg seed, scale)
CASES = [
    ("append_m1_off5", 14, 2, 64, 5, 1, 16, 0, 1, 1.0),       # tests/kv_prep_fused.rs:249-267
    ("append_m4_off0", 14, 2, 64, 0, 4, 16, 1, 7, 1.0),
    ("append_m2_d128", 32, 8, 128, 0, 2, 64, 0, 42, 1.0),
    ("decode_d64_l128", 14, 14, 64, 127, 1, 128, 0, 1, 0.25),  # tests/flashattention_decode_parity.rs
    ("decode_d128_l128", 8, 8, 128, 127, 1, 128, 0, 7, 0.25),
    ("decode_d64_l27", 14, 14, 64, 26, 1, 64, 0, 42, 0.25),
    ("decode_gqa_d64", 14, 2, 64, 99, 1, 128, 0, 11, 0.25),
    ("prefill_m17_d64", 14, 14, 64, 0, 17, 32, 0, 19, 0.25),   # tests/flashattention_prefill_parity.rs
    ("prefill_m32_prefix64_d128", 8, 8, 128, 64, 32, 96, 0, 29, 0.25),
    ("prefill_m26_gqa", 14, 2, 64, 64, 26, 128, 1, 41, 0.25),
]


def build(name, hq, hkv, d, cached, m, cap, mode, seed, scale):
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=cached, m=m, capacity=cap, theta=1e4,
                      rope_mode=mode, gen="lcg", seed=seed, scale=scale)
    q_rot, kc, vc = case.oracle_append()
    out = {f"{name}/q_rot": q_rot, f"{name}/k_rows": kc[:, cached:cached + m].copy(),
           f"{name}/v_rows": vc[:, cached:cached + m].copy()}
    if name.startswith("decode"):
        out[f"{name}/out"] = oracle.decode_online(q_rot, kc, vc, n_heads=hq, cache_heads=hkv, head_dim=d, capacity=cap,
                                                  kv_len=cached + m, scale=case.scale)
    if name.startswith("prefill"):
        out[f"{name}/out"] = oracle.prefill_causal(q_rot, kc, vc, n_heads=hq, cache_heads=hkv, head_dim=d,
                                                   capacity=cap, q_len=m, kv_len=cached + m, query_offset=cached,
                                                   scale=case.scale)
    return out


# Fused QKV projection (name, m, k_dim, n_dim, n_kv, gamma, bias, weights_per_block, lcg seed): the
# shapes of the reference's tests/fused_qkv_batched_rmsnorm_parity.rs:58-66 and tests/qkv_parity_f16.rs:87-89
QKV_CASES = [
    ("qkv_m2_k128_blocked", 2, 128, 128, 64, True, False, 32, 3),
    ("qkv_m1_k1024_rowmajor_bias", 1, 1024, 1024, 128, True, True, 0, 5),
]


def qkv_inputs(m, k_dim, n_dim, n_kv, gamma, bias, wpb, seed):
    """Deterministic inputs: activations in [-1, 1), weights and biases in [-0.1, 0.1), gamma in [0.5, 1.5)."""
    st = seed
    x, st = oracle.lcg_fill(st, m * k_dim, 1.0)
    ws = []
    for n in (n_dim, n_kv, n_kv):
        w, st = oracle.lcg_fill(st, n * k_dim, 0.1)
        ws.append(w)
    g = None
    if gamma:
        g, st = oracle.lcg_fill(st, k_dim, 0.5)
        g = (g.view(np.float16).astype(np.float32) + 1.0).astype(np.float16).view(np.uint16)
    bs = [None] * 3
    if bias:
        bs = []
        for n in (n_dim, n_kv, n_kv):
            b, st = oracle.lcg_fill(st, n, 0.1)
            bs.append(b)
    return x, ws, g, bs


def build_qkv(name, m, k_dim, n_dim, n_kv, gamma, bias, wpb, seed):
    x, ws, g, bs = qkv_inputs(m, k_dim, n_dim, n_kv, gamma, bias, wpb, seed)
    if wpb:  # row-major [n, k] -> the reference's blocked layout
        ws = [np.ascontiguousarray(w.reshape(n, k_dim // wpb, wpb).transpose(1, 0, 2)).ravel()
              for w, n in zip(ws, (n_dim, n_kv, n_kv))]
    q, k, v = oracle.fused_qkv(x, *ws, m=m, k_dim=k_dim, n_dim=n_dim, n_kv=n_kv, gamma=g, b_q=bs[0], b_k=bs[1],
                               b_v=bs[2], weights_per_block=wpb)
    return {f"{name}/q": q, f"{name}/k": k, f"{name}/v": v}


def main():
    data = {}
    for c in CASES:
        data.update(build(*c))
    for c in QKV_CASES:
        data.update(build_qkv(*c))
    cos, sin = oracle.rope_tables(1e6, 64, 512)
    data["rope_1e6_d64/cos_rows"] = cos[[0, 1, 2, 255, 511]]
    data["rope_1e6_d64/sin_rows"] = sin[[0, 1, 2, 255, 511]]
    cos, sin = oracle.rope_tables(5e5, 128, 8192)
    data["rope_5e5_d128/cos_rows"] = cos[[1, 4095, 8191]]
    data["rope_5e5_d128/sin_rows"] = sin[[1, 4095, 8191]]
    data["lcg_seed1_scale025"] = oracle.lcg_fill(1, 256, 0.25)[0]
    data["normal_seed5EED_t1"] = oracle.normal_fill(0x5EED, 1, 256)
    np.savez_compressed(Path(__file__).with_name("kv_path_golden.npz"), **data)
    print(f"wrote {len(data)} arrays")


if __name__ == "__main__":
    main()
