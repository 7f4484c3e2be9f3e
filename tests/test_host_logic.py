"""CPU tests (no GPU): the C ABI loads and exports every declared symbol, the host-side logic
gives the reference's known answers, and the step planner keeps its invariants."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "metallic_cuda.h").read_text()
    return sorted(set(re.findall(r"MF_API\s+[\w\s\*]+?\b(mf_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(mfk):
    names = declared_symbols()
    assert len(names) >= 35
    for n in names:
        assert hasattr(mfk.lib, n), f"{n} is declared in include/metallic_cuda.h but not exported"
    assert sorted(mfk.EXPORTED_SYMBOLS) == names, "the Python binding must cover exactly the declared symbols"
    assert mfk.lib.mf_abi_version() == 1


def test_no_cpu_fallback(mfk):
    """Without an sm_100 device a context cannot be created; nothing computes on the CPU."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(mfk.MetalError):
        mfk.Foundry()


def test_param_struct_layouts(mfk):
    """The #[repr(C)] parameter structs are plain 4-byte fields with no padding."""
    assert C.sizeof(mfk.KvPrepFusedParamsResolved) == 13 * 4  # kv_prep/mod.rs:79-114
    assert C.sizeof(mfk.RopeParamsResolved) == 4 * 4          # rope/mod.rs:11-22
    assert C.sizeof(mfk.KvCacheWriteParamsResolved) == 7 * 4  # kv_cache_write/mod.rs:61-78
    assert C.sizeof(mfk.KvCacheWriteRepeatKvHeadsParamsResolved) == 9 * 4
    assert C.sizeof(mfk.SdpaParams) == 5 * 4                  # flashattention/stages.rs:456-464
    assert C.sizeof(mfk.SdpaPrefillParams) == 18 * 4          # stages.rs:240-270
    assert C.sizeof(mfk.SdpaPrefillSplitKParams) == 20 * 4    # stages.rs:272-306
    assert mfk.SdpaParams.scale.offset == 8 and mfk.SdpaPrefillParams.query_offset.offset == 20
    assert mfk.KvPrepFusedParamsResolved.rope_mode.offset == 40
    assert C.sizeof(mfk.MfTensor) == 8 + 8 + 4 + 4 + 32 + 32


def test_align_capacity_known_answers(mfk):
    """ContextConfig::align_capacity test (src/model/context.rs:308-316)."""
    for n, want in [(0, 128), (1, 128), (127, 128), (128, 128), (129, 256), (200, 256)]:
        assert mfk.align_capacity(n) == want


def test_memory_estimate_known_answer(mfk):
    """test_memory_estimation (src/model/context.rs:318-324): 4 layers, 2 kv heads, D 64, ctx 2048."""
    assert mfk.lib.mf_estimate_kv_memory(4, 2, 64, 2048) == 4194304
    # per_token_bytes_f16 (kv_geometry.rs:82-89) for Llama-3.2-3B compact: 28 * 2 * 8 * 128 * 2
    assert mfk.lib.mf_kv_per_token_bytes_f16(28, 8, 128) == 28 * 2 * 8 * 128 * 2
    # configuration 2: 28 layers of [8, 8192, 128] f16 K and V = 896 MiB
    assert mfk.lib.mf_estimate_kv_memory(28, 8, 128, 8192) == 896 * 1024 * 1024


def test_growth_rule(mfk):
    """ensure_kv_capacity (src/model/executor.rs:2332-2396): keep, double, clamp, align."""
    assert mfk.grown_capacity(2048, 100, 8192) == 2048          # already sufficient
    assert mfk.grown_capacity(2048, 2049, 8192) == 4096         # x2
    assert mfk.grown_capacity(2048, 5000, 8192) == 5120         # required > 2x, aligned to 128
    assert mfk.grown_capacity(4096, 4097, 6000) == 6016         # clamped to max, then aligned
    assert mfk.grown_capacity(2048, 9000, 8192) == 0            # exceeds the context limit


def test_prefill_split_k_heuristic(mfk):
    """src/metals/flashattention/step.rs:849-866."""
    assert mfk.prefill_split_k(4096, 2048) == 8
    assert mfk.prefill_split_k(4096, 16) == 8
    assert mfk.prefill_split_k(4096, 15) == 1
    assert mfk.prefill_split_k(2048, 64) == 4
    assert mfk.prefill_split_k(2047, 64) == 1
    assert mfk.prefill_split_k(1024, 32) == 1
    assert mfk.prefill_split_k(33, 33) == 1


def test_rope_tables_match_oracle(mfk, orc):
    for theta, d, n in [(1e4, 64, 64), (1e6, 64, 512), (5e5, 128, 300)]:
        cos, sin = mfk.rope_tables(theta, d, n)
        c2, s2 = orc.rope_tables(theta, d, n)
        assert np.array_equal(cos, c2) and np.array_equal(sin, s2)
    ff = np.linspace(1, 4, 64).astype(np.float32)
    cos, sin = mfk.rope_tables(5e5, 128, 40, first_pos=1000, freq_factors=ff)
    c2, s2 = orc.rope_tables(5e5, 128, 40, first_pos=1000, freq_factors=ff)
    assert np.array_equal(cos, c2) and np.array_equal(sin, s2)


def check_plan(items, cta_begin, kv_lens, n_kv_heads, max_ctas):
    tiles = (np.asarray(kv_lens, np.int64) + 63) // 64
    total = int(tiles.sum()) * n_kv_heads
    n_ctas = len(cta_begin) - 1
    assert n_ctas == min(max_ctas, total) or total == 0
    if total == 0:
        assert len(items) == 0
        return
    assert cta_begin[0] == 0 and cta_begin[-1] == len(items) and np.all(np.diff(cta_begin) >= 0)
    per_cta = [int(sum(items[i, 3] - items[i, 2] for i in range(cta_begin[c], cta_begin[c + 1]))) for c in range(n_ctas)]
    assert sum(per_cta) == total
    one_item_per_cta = len(items) == n_ctas and np.array_equal(cta_begin, np.arange(n_ctas + 1))
    if not one_item_per_cta:
        # long launches: what is equal is tiles + ITEM_COST * pieces (a piece of a unit costs its CTA the staging of q,
        # a combine, a partial and a ticket); no CTA is more than one piece and a minimum piece above the mean
        ITEM_COST, MIN_PIECE = 20, 4
        cost = np.array([t + ITEM_COST * (cta_begin[c + 1] - cta_begin[c]) for c, t in enumerate(per_cta)])
        assert cost.max() <= cost.sum() / n_ctas + ITEM_COST + MIN_PIECE + 1
        assert cost.max() <= np.median(cost) + ITEM_COST + MIN_PIECE + 1
    # every (sequence, kv head) unit is covered exactly once, in order, by consecutive slots
    seen = {}
    for i, (seq, kvh, tb, te, slot, unit, n_parts, first_slot) in enumerate(items.tolist()):
        assert te > tb and unit == seq * n_kv_heads + kvh and slot == i
        cov = seen.setdefault(unit, [])
        assert tb == (cov[-1][1] if cov else 0)
        cov.append((tb, te))
        assert first_slot == slot - (len(cov) - 1)
    for unit, cov in seen.items():
        assert cov[-1][1] == tiles[unit // n_kv_heads]
        assert all(items[i, 6] == len(cov) for i in range(len(items)) if items[i, 5] == unit)
    assert len(seen) == int((tiles > 0).sum()) * n_kv_heads


@pytest.mark.parametrize("seed", range(8))
def test_cluster_plans_for_sequences_of_different_lengths(mfk, seed):
    """Short launches (at most one CTA per SM) over sequences of different lengths: clusters of one size, every unit cut
    into ranges of about equal length, one cluster per range.  Every range has at least one tile per CTA of its
    cluster, the ranges of a unit cover it in order, the CTAs fit the launch, and clusters of 16 are only used when
    no unit needs a second range."""
    rng = np.random.default_rng(100 + seed)
    batch = int(rng.integers(1, 10))
    n_kv_heads = int(rng.choice([1, 2, 8]))
    lens = rng.integers(512, 16385, size=batch).astype(np.uint32)
    if seed == 0:
        lens[:] = 8192                      # equal lengths: the uniform cluster plan
    if seed == 1:
        lens[0] = 0                         # a sequence without keys has no unit
    max_ctas = 148
    fit16, fit8 = (14, 36) if seed % 2 else (0, 0)
    items, cluster = mfk.build_decode_plan_host_clusters(lens, n_kv_heads, max_ctas, 16, fit16, fit8)
    tiles = (lens.astype(np.int64) + 63) // 64
    total = int(tiles.sum()) * n_kv_heads
    if cluster == 0:                        # plain form: the other planner's invariants
        plain, cta_begin = mfk.build_decode_plan_host(lens, n_kv_heads, max_ctas)
        assert np.array_equal(items, plain)
        check_plan(plain, cta_begin, lens, n_kv_heads, max_ctas)
        return
    assert cluster in (2, 4, 8, 16) and len(items) * cluster <= max_ctas
    if cluster == 16 and fit16:
        assert len(items) <= fit16
    if cluster == 8 and fit8:
        assert len(items) <= fit8
    uniform = len(set(int(t) for t in tiles if t)) == 1   # equal lengths: ranges of ceil(T / k) tiles, the last one shorter
    seen = {}
    for i, (seq, kvh, tb, te, slot, unit, n_parts, first_slot) in enumerate(items.tolist()):
        assert te - tb >= (1 if uniform else cluster) and unit == seq * n_kv_heads + kvh and slot == i
        cov = seen.setdefault(unit, [])
        assert tb == (cov[-1][1] if cov else 0)
        cov.append((tb, te))
        assert first_slot == slot - (len(cov) - 1)
    for unit, cov in seen.items():
        assert cov[-1][1] == tiles[unit // n_kv_heads]
        assert all(items[i, 6] == len(cov) for i in range(len(items)) if items[i, 5] == unit)
        spans = [e - b for b, e in cov]
        if uniform:
            assert all(x == spans[0] for x in spans[:-1]) and spans[-1] <= spans[0]
        else:
            assert max(spans) - min(spans) <= 1       # ranges of equal length
            if cluster == 16:
                assert len(cov) == 1
    assert len(seen) == int((tiles > 0).sum()) * n_kv_heads
    assert sum(e - b for cov in seen.values() for b, e in cov) == total


@pytest.mark.parametrize("seed", range(6))
def test_decode_plan_invariants(mfk, seed):
    rng = np.random.default_rng(seed)
    batch = int(rng.integers(1, 70))
    lens = rng.integers(0, 20000, size=batch).astype(np.uint32)
    if seed == 0:
        lens[:] = 0
    if seed == 1:
        lens = np.array([1], np.uint32)
    for n_kv_heads, max_ctas in [(2, 148), (8, 296), (1, 7), (2, 100000)]:
        items, cta_begin = mfk.build_decode_plan_host(lens, n_kv_heads, max_ctas)
        check_plan(items, cta_begin, lens, n_kv_heads, max_ctas)


def test_decode_plan_c3_shape(mfk):
    rng = np.random.default_rng(0x5EED)
    lens = rng.integers(512, 16385, size=64).astype(np.uint32) + 1
    items, cta_begin = mfk.build_decode_plan_host(lens, 2, 296)
    check_plan(items, cta_begin, lens, 2, 296)
    assert len(items) <= 128 + 296


@pytest.mark.parametrize("lens,n_kv_heads,max_ctas", [([8192], 8, 148), ([131072 // 8], 8, 296), ([100, 900, 2000], 2, 148),
                                                       ([4097, 4100], 4, 148)])
def test_decode_plan_cuts_units_separately_when_the_launch_is_short(mfk, lens, n_kv_heads, max_ctas):
    """Few tiles per CTA and several CTAs per unit: no CTA straddles two (sequence, kv head) units (a
    straddling CTA pays the per-item work twice and the launch ends with the slowest CTA)."""
    lens = np.array(lens, np.uint32)
    items, cta_begin = mfk.build_decode_plan_host(lens, n_kv_heads, max_ctas)
    tiles = (lens.astype(np.int64) + 63) // 64
    n_ctas = len(cta_begin) - 1
    assert n_ctas <= max_ctas and len(items) == n_ctas
    assert np.array_equal(cta_begin, np.arange(n_ctas + 1))  # one item per CTA
    seen = {}
    for i, (seq, kvh, tb, te, slot, unit, n_parts, first_slot) in enumerate(items.tolist()):
        assert te > tb and unit == seq * n_kv_heads + kvh and slot == i
        cov = seen.setdefault(unit, [])
        assert tb == (cov[-1][1] if cov else 0) and first_slot == slot - len(cov)
        cov.append((tb, te))
    assert len(seen) == len(lens) * n_kv_heads
    for unit, cov in seen.items():
        assert cov[-1][1] == tiles[unit // n_kv_heads]
        sizes = [b - a for a, b in cov]
        assert max(sizes) - min(sizes) <= 1
        assert all(items[i, 6] == len(cov) for i in range(len(items)) if items[i, 5] == unit)
    # longest range within one tile of the ideal
    assert max(items[:, 3] - items[:, 2]) <= -(-int(tiles.sum()) * n_kv_heads // n_ctas) + 1


def _ctx_cfg(mfk, model_max, override=0, env_cap=0, full_reserve=0, budget_mb=-1):
    cfg = mfk.MfContextConfig()
    assert mfk.lib.mf_context_config_from_architecture(model_max, override, env_cap, full_reserve, budget_mb, C.byref(cfg)) == 0
    return cfg


def test_context_config_priority_known_answers(mfk):
    """test_context_config_priority (src/model/context.rs:288-305) and the rules of from_architecture (:105-152)."""
    assert _ctx_cfg(mfk, 4096).max_context_len == 4096                      # 1. defaults to the model max
    assert _ctx_cfg(mfk, 4096, override=2048).max_context_len == 2048       # 2. the caller's value is a cap
    assert _ctx_cfg(mfk, 4096, env_cap=1024).max_context_len == 1024        # 3. so is the environment's
    assert _ctx_cfg(mfk, 4096, override=2048, env_cap=1024).max_context_len == 2048  # the caller's wins over the env
    assert _ctx_cfg(mfk, 4096, override=100000).max_context_len == 4096     # never beyond the model
    assert _ctx_cfg(mfk, 0, override=3000).max_context_len == 3000          # no model max: the cap
    assert _ctx_cfg(mfk, 0).max_context_len == 2048                         # neither: 2048
    c = _ctx_cfg(mfk, 32768)
    assert (c.allocated_capacity, c.full_reserve, c.budget_bytes) == (2048, 0, 0) and abs(c.budget_auto_pct - 0.5) < 1e-7
    assert _ctx_cfg(mfk, 1000).allocated_capacity == 1024                   # align(min(2048, max))
    assert _ctx_cfg(mfk, 32768, full_reserve=1).allocated_capacity == 32768
    c = _ctx_cfg(mfk, 32768, budget_mb=64)
    assert c.budget_bytes == 64 << 20 and c.budget_auto_pct == 0.0


def test_context_config_reads_the_reference_environment(mfk, monkeypatch):
    monkeypatch.setenv("METALLIC_MAX_CONTEXT_LEN", " 1024 ")  # trimmed, as the reference does (:107-109)
    monkeypatch.setenv("METALLIC_FULL_CONTEXT_RESERVE", "1")
    monkeypatch.setenv("METALLIC_KV_MEMORY_BUDGET_MB", "8")
    cfg = mfk.MfContextConfig()
    assert mfk.lib.mf_context_config_from_env(4096, 0, C.byref(cfg)) == 0
    assert (cfg.max_context_len, cfg.allocated_capacity, cfg.full_reserve, cfg.budget_bytes) == (1024, 1024, 1, 8 << 20)
    monkeypatch.setenv("METALLIC_MAX_CONTEXT_LEN", "not a number")  # parse failure = unset
    monkeypatch.delenv("METALLIC_FULL_CONTEXT_RESERVE")
    assert mfk.lib.mf_context_config_from_env(4096, 0, C.byref(cfg)) == 0
    assert (cfg.max_context_len, cfg.allocated_capacity, cfg.full_reserve) == (4096, 2048, 0)


def test_apply_memory_budget(mfk):
    """apply_memory_budget (src/model/context.rs:158-210): budget / per_token_bytes, aligned to 128, floor of 1."""
    per_token = mfk.lib.mf_kv_per_token_bytes_f16(28, 8, 128)  # Llama-3.2-3B compact: 114 688 B per token
    assert per_token == 28 * 2 * 8 * 128 * 2
    cfg = _ctx_cfg(mfk, 131072, full_reserve=1, budget_mb=1024)  # 1 GiB / 114 688 = 9362 tokens -> 9472
    assert mfk.lib.mf_apply_memory_budget(C.byref(cfg), 0, per_token) == 0
    assert (cfg.max_context_len, cfg.allocated_capacity) == (9472, 9472)
    cfg = _ctx_cfg(mfk, 8192, budget_mb=1024)                    # the budget allows more than the model: unchanged
    mfk.lib.mf_apply_memory_budget(C.byref(cfg), 0, per_token)
    assert (cfg.max_context_len, cfg.allocated_capacity) == (8192, 2048)
    cfg = _ctx_cfg(mfk, 8192)                                    # Auto 50 % of the device figure
    mfk.lib.mf_apply_memory_budget(C.byref(cfg), 2 * 4096 * per_token, per_token)
    assert (cfg.max_context_len, cfg.allocated_capacity) == (4096, 2048)
    cfg = _ctx_cfg(mfk, 8192, budget_mb=0)                       # a zero budget changes nothing (:186-188)
    mfk.lib.mf_apply_memory_budget(C.byref(cfg), 0, per_token)
    assert cfg.max_context_len == 8192
    cfg = _ctx_cfg(mfk, 8192)                                    # too small for one token: pinned to 1 / 128
    mfk.lib.mf_apply_memory_budget(C.byref(cfg), per_token, per_token)  # 50 % of one token
    assert (cfg.max_context_len, cfg.allocated_capacity) == (1, 128)


def test_kv_geometry_known_answers(mfk):
    """kv_geometry_compact_defaults_for_gqa (src/model/kv_geometry.rs:221-230) and the clamps of :26-36."""
    g = mfk.MfKvGeometry()
    assert mfk.lib.mf_kv_geometry_from_architecture(24, 8, 3072, C.byref(g)) == 0
    assert (g.layout, g.n_heads, g.n_kv_heads, g.group_size, g.head_dim, g.cache_heads) == (
        mfk.KV_LAYOUT_COMPACT_KV_HEADS, 24, 8, 3, 128, 8)
    mfk.lib.mf_kv_geometry_from_architecture(8, 0, 512, C.byref(g))    # no kv head count: MHA, expanded
    assert (g.n_kv_heads, g.group_size, g.layout, g.cache_heads) == (8, 1, 0, 8)
    mfk.lib.mf_kv_geometry_from_architecture(8, 16, 512, C.byref(g))   # clamped to n_heads
    assert g.n_kv_heads == 8
    mfk.lib.mf_kv_geometry_from_architecture(14, 4, 896, C.byref(g))   # does not divide: group 1
    assert (g.group_size, g.layout, g.cache_heads) == (1, 1, 4)


def test_kv_geometry_from_cache_tensor(mfk):
    """from_cache_tensor (src/model/kv_geometry.rs:92-150): layout from the head count, four refusals."""
    def tensor(dims, dtype=0):
        t = mfk.MfTensor()
        t.dev_ptr, t.offset_bytes, t.dtype, t.rank = 0x1000, 0, dtype, len(dims)
        for i, d in enumerate(dims):
            t.dims[i] = d
        return t

    g, err = mfk.MfKvGeometry(), C.create_string_buffer(256)
    call = lambda t, cap=8192: mfk.lib.mf_kv_geometry_from_cache_tensor(24, 8, 3072, C.byref(t), cap, C.byref(g), err, 256)
    assert call(tensor([8, 8192, 128])) == 0 and (g.layout, g.cache_heads) == (1, 8)
    assert call(tensor([24, 8192, 128])) == 0 and (g.layout, g.cache_heads) == (0, 24)
    INVALID_SHAPE = 2
    assert call(tensor([8, 8192, 128], dtype=1)) == INVALID_SHAPE and b"must be F16" in err.value
    assert call(tensor([8, 8192])) == INVALID_SHAPE and b"rank-3" in err.value
    assert call(tensor([8, 4096, 128])) == INVALID_SHAPE and err.value == b"KV cache capacity mismatch: got 4096, expected 8192"
    assert call(tensor([8, 8192, 64])) == INVALID_SHAPE and err.value == b"KV cache head_dim mismatch: got 64, expected 128"
    assert call(tensor([12, 8192, 128])) == INVALID_SHAPE
    assert err.value == b"KV cache heads mismatch: got 12, expected 24 (expanded) or 8 (compact)"
