"""Pins the CPU oracle against what the reference's own tests pin.

The reference stores no numeric golden outputs for the routed-expert path; its
tests regenerate inputs from seeds and compare two implementations. So the
oracle is pinned by (a) the literal grouping vectors, (b) struct layouts,
(c) the published SplitMix64 / FNV-1a algorithms, (d) the relations the
reference's tests assert, on the reference's seeds, shapes and tolerances.
"""
import ctypes as C
import json
from pathlib import Path

import numpy as np
import pytest

GOLDEN = Path(__file__).parent / "golden"


def _pairs(o, rows):
    a = np.zeros(len(rows), dtype=o.PAIR_DTYPE)
    for i, (t, e, r, w) in enumerate(rows):
        a[i] = (t, e, r, w)
    return a


# ---- (a) grouping known-answer vectors ------------------------------------

def _check_grouping_case(o, group_fn, case):
    rows = case["pairs"]
    if case.get("pairs_reversed"):
        rows = rows[::-1]
    g = group_fn(_pairs(o, rows), case["query_count"], case["top_k"], case["num_experts"],
                 case["tile_expert_count"], case["sort_keys"])
    sp = g.sorted_pairs
    if "sorted_experts" in case:
        assert sp["expert"].tolist() == case["sorted_experts"]
    if "sorted_token_rank" in case:
        assert [[int(t), int(r)] for t, r in zip(sp["token"], sp["rank"])] == case["sorted_token_rank"]
    if "sorted_weight_bits" in case:
        assert sp[sp.dtype.names[3]].tolist() == case["sorted_weight_bits"]
    if "per_expert_offsets" in case:
        assert g.per_expert_offsets.tolist() == case["per_expert_offsets"]
    if "per_expert_counts" in case:
        assert g.per_expert_counts.tolist() == case["per_expert_counts"]
    if "groups" in case:
        assert [list(map(int, x)) for x in g.groups.tolist()] == case["groups"]
    if "group_experts" in case:
        assert g.groups["expert"].tolist() == case["group_experts"]
    if "tiles" in case:
        assert [list(map(int, x)) for x in g.tiles.tolist()] == case["tiles"]
    if "shuffle" in case:
        shuffled = [case["pairs"][i] for i in case["shuffle"]]
        g2 = group_fn(_pairs(o, shuffled), case["query_count"], case["top_k"], case["num_experts"],
                      case["tile_expert_count"], case["sort_keys"])
        assert g2.sorted_pairs.tobytes() == sp.tobytes()
        assert g2.groups.tobytes() == g.groups.tobytes() and g2.tiles.tobytes() == g.tiles.tobytes()
    if "max_pairs_per_expert" in case:
        assert int(g.groups["pair_count"].max()) == case["max_pairs_per_expert"]
        assert int(g.tiles["pair_count"].max()) == case["max_pairs_per_tile"]
        assert int(g.tiles["group_count"].max()) == case["max_live_experts_per_tile"]
    for tile in g.tiles:   # pair ranges stay contiguous per tile
        sl = sp[int(tile["pair_start"]):int(tile["pair_start"] + tile["pair_count"])]
        ex = g.groups[int(tile["group_start"]):int(tile["group_start"] + tile["group_count"])]["expert"]
        assert set(sl["expert"].tolist()) == set(ex.tolist())


def test_grouping_known_answers(oracle):
    data = json.loads((GOLDEN / "grouping_vectors.json").read_text())
    for case in data["cases"]:
        _check_grouping_case(oracle, oracle.group_pairs, case)


def test_grouping_rejects_invalid_metadata(oracle):
    data = json.loads((GOLDEN / "grouping_vectors.json").read_text())
    for err in data["errors"]:
        with pytest.raises(oracle.GroupingError) as ei:
            oracle.group_pairs(_pairs(oracle, err["pairs"]), err["query_count"], err["top_k"], err["num_experts"],
                               err["tile_expert_count"], err["sort_keys"])
        assert ei.value.case == err["case"]


def test_grouping_real_trace_pressure_t32(oracle):
    # PrefillMoEGroupingTests.swift:175-205
    rows = [[t, (t + r * 7) % 74, r, t * 8 + r] for t in range(32) for r in range(8)]
    g = oracle.group_pairs(_pairs(oracle, rows), 32, 8, 128, 16)
    assert len(g.sorted_pairs) == 256 and len(g.groups) <= 74
    assert int(g.tiles["group_count"].max()) <= 16 and int(g.tiles["pair_count"].max()) <= 256
    assert (g.tiles["pair_count"] > 0).all()


def test_make_token_expert_pairs_is_token_major(oracle):
    idx = np.array([[3, 1], [0, 2]], dtype=np.uint32)
    w = oracle.f32_to_f16(np.array([[0.5, 0.25], [0.75, 0.125]], dtype=np.float32))
    p = oracle.make_token_expert_pairs(idx, w, 2, 2)
    assert p["token"].tolist() == [0, 0, 1, 1] and p["rank"].tolist() == [0, 1, 0, 1]
    assert p["expert"].tolist() == [3, 1, 0, 2]
    assert p["weight_bits"].tolist() == [0x3800, 0x3400, 0x3A00, 0x3000]


# ---- (b) layouts -------------------------------------------------------------

def test_struct_layouts(oracle):
    # PrefillRouterTests.swift:12-19 (16-byte pair, fields at 0/4/8/12); MoE.swift:4-29 (9 x u32)
    assert oracle.PAIR_DTYPE.itemsize == 16
    assert [oracle.PAIR_DTYPE.fields[n][1] for n in oracle.PAIR_DTYPE.names] == [0, 4, 8, 12]
    assert C.sizeof(oracle.ExpertOffsets) == 36


def test_production_blob_layout(oracle):
    # RepackPlanner.swift:337-399 / docs/SYSTEM_DESIGN.md:166
    off, payload, stride = oracle.blob_layout(2816, 704)
    assert [getattr(off, n) for n, _ in off._fields_] == [0, 991232, 1053184, 1115136, 2106368, 2168320,
                                                          2230272, 3221504, 3283456]
    assert payload == 3345408 and stride == 3358720


# ---- (c) PRNG and 16-bit conversions ---------------------------------------------

def test_splitmix64_published_vectors(oracle):
    # First outputs of SplitMix64 from seed 0 and the widely quoted seed 1234567
    # stream (Vigna's reference implementation).
    r = oracle.SplitMix64(0)
    assert r.next() == 0xE220A8397B1DCDAF
    assert r.next() == 0x6E789E6AA1B965F4
    r = oracle.SplitMix64(1234567)
    assert [r.next() for _ in range(2)] == [6457827717110365317, 3203168211198807973]


def test_uniform_is_24_bit(oracle):
    r = oracle.SplitMix64(0xA5B61234)
    raw = oracle.SplitMix64(0xA5B61234).next()
    assert r.uniform(-1.0, 1.0) == np.float32(-1.0) + np.float32(2.0) * (np.float32(raw >> 40) / np.float32(1 << 24))


def test_seedtree_fnv1a(oracle):
    # FNV-1a 64 of "a" is 0xaf63dc4c8601ec8c (published test vector); the key is root ^ hash.
    assert oracle.lib().tfo_seedtree_key(0, b"a") == 0xAF63DC4C8601EC8C
    assert oracle.lib().tfo_seedtree_key(0xFF, b"") == 0xCBF29CE484222325 ^ 0xFF


def test_bf16_round_half_even(oracle):
    l = oracle.lib()
    assert l.tfo_bf16_bits(1.0) == 0x3F80
    assert l.tfo_bf16_bits(np.float32(np.frombuffer(np.uint32(0x3F808000).tobytes(), np.float32)[0])) == 0x3F80  # tie -> even
    assert l.tfo_bf16_bits(np.float32(np.frombuffer(np.uint32(0x3F818000).tobytes(), np.float32)[0])) == 0x3F82  # tie -> even (up)
    assert l.tfo_bf16_bits(np.float32(np.frombuffer(np.uint32(0x3F808001).tobytes(), np.float32)[0])) == 0x3F81
    assert l.tfo_bf16_to_float(0x3F80) == 1.0


def test_fp16_conversion_matches_ieee(oracle):
    rng = np.random.default_rng(7)
    vals = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * 10,
        rng.standard_normal(5000).astype(np.float32) * 1e-5,       # subnormals
        np.array([0.0, -0.0, 65504.0, 65520.0, 1e6, -1e6, 6.1e-5, 5.96e-8, 2.98e-8, 2.99e-8], dtype=np.float32),
    ])
    ours = oracle.f32_to_f16(vals)
    ref = vals.astype(np.float16).view(np.uint16)
    assert np.array_equal(ours, ref)
    all_bits = np.arange(0, 0x7C00, dtype=np.uint16)
    assert np.array_equal(oracle.f16_to_f32(all_bits), all_bits.view(np.float16).astype(np.float32))


# ---- (d) relations the reference's tests assert --------------------------------------

def test_int4_round_trip_bound(oracle):
    # QuantizationTests.swift:8-34
    rng = oracle.SeedTree(0x51A71001).key("int4-affine-round-trip")
    row = rng.uniform_array(-1.0, 1.0, 256)
    q = oracle.quantize_rows(row[None, :], 4)
    r = oracle.dequantize(q)[0]
    for g in range(4):
        amax = np.abs(row[g * 64:(g + 1) * 64]).max()
        assert np.all(np.abs(r[g * 64:(g + 1) * 64] - row[g * 64:(g + 1) * 64]) <= amax / 7.0 + 1e-3)


def test_nibble_layout_low_even_high_odd(oracle):
    # QuantizationTests.swift:36-50
    row = (np.arange(64, dtype=np.float32) - 31.5)[None, :]
    q = oracle.quantize_rows(row, 4)
    b0 = int(q.packed[0, 0])
    scale = oracle.bf16_to_f32(q.scales[0, :1])[0]
    bias = oracle.bf16_to_f32(q.biases[0, :1])[0]
    assert abs((b0 & 0xF) * scale + bias - row[0, 0]) <= scale + 1e-3
    assert abs((b0 >> 4) * scale + bias - row[0, 1]) <= scale + 1e-3
    # codes must be monotone over an increasing ramp, low nibble first
    codes = np.stack([q.packed[0] & 0xF, q.packed[0] >> 4], axis=1).reshape(-1)
    assert np.all(np.diff(codes.astype(int)) >= 0) and codes[0] == 0 and codes[-1] == 15


def test_constant_group_is_exact(oracle):
    row = np.full((1, 64), 0.375, dtype=np.float32)
    for bits in (4, 8):
        q = oracle.quantize_rows(row, bits)
        assert np.array_equal(oracle.dequantize(q), row)


@pytest.mark.parametrize("m,n,seed,label", [
    (128, 128, 0xC1, "int4-gemv-kernel-m128-n128"),
    (1024, 2816, 0xC2, "int4-gemv-kernel-m1024-n2816"),
    (64, 64, 0xC3, "int4-gemv-kernel-m64-n64"),
    (128, 2816, 0xC4, "int4-gemv-kernel-m128-n2816-off2"),
])
def test_int4_gemv_kernel_order_vs_dequant_reference(oracle, m, n, seed, label):
    # DequantInt4GEMVTests.swift:41-121: rel < Tolerance.fp16Reduction (5e-3)
    rng = oracle.SeedTree(seed).key(label)
    rows = np.stack([rng.uniform_array(-0.5, 0.5, n) for _ in range(m)])
    mat = oracle.quantize_rows(rows, 4)
    x16 = oracle.f32_to_f16(rng.uniform_array(-1.0, 1.0, n))
    ref = oracle.gemv_ref(mat, oracle.f16_to_f32(x16))
    y16, y32 = oracle.gemv_kernel_order(mat, x16)
    assert oracle.rel_error(oracle.f16_to_f32(y16), ref) < 5e-3
    assert oracle.rel_error(y32, ref) < 1e-5
    assert oracle.rel_error(oracle.gemv_ref(mat, oracle.f16_to_f32(x16), acc="f32"), ref) < 1e-5


@pytest.mark.parametrize("m,n,seed", [(128, 2816, 0x151), (1024, 2816, 0x152)])
def test_int8_gemv_kernel_order_vs_dequant_reference(oracle, m, n, seed):
    # DequantInt8GEMVTests.swift:74-88
    rng = oracle.SplitMix64(seed)
    rows = np.stack([rng.uniform_array(-0.5, 0.5, n) for _ in range(m)])
    mat = oracle.quantize_rows(rows, 8)
    x16 = oracle.f32_to_f16(rng.uniform_array(-1.0, 1.0, n))
    ref = oracle.gemv_ref(mat, oracle.f16_to_f32(x16))
    y16, y32 = oracle.gemv_kernel_order(mat, x16)
    assert oracle.rel_error(oracle.f16_to_f32(y16), ref) < 5e-3
    assert oracle.rel_error(y32, ref) < 1e-5


def _router_fixture(o, seed=0xA5B61234, experts=16, dim=128):
    # RouterTopKTests.swift:17-45
    rng = o.SplitMix64(seed)
    weights = np.stack([rng.uniform_array(-0.05, 0.05, dim) + np.float32(e) * np.float32(0.01) for e in range(experts)])
    hidden = rng.uniform_array(-1.0, 1.0, dim)
    inv = np.float32(1.0) / np.sqrt(np.float32(dim))
    eff = rng.uniform_array(0.5, 1.5, dim) * inv
    gain = rng.uniform_array(0.6, 1.4, experts)
    return weights, hidden, eff, gain


def test_router_matches_sorted_reference(oracle):
    o = oracle
    weights, hidden, eff, gain = _router_fixture(o)
    mat = o.quantize_rows(weights, 8)
    h16, e16, g16 = o.f32_to_f16(hidden), o.f32_to_bf16(eff), o.f32_to_bf16(gain)
    logits = o.router_logits(mat, h16, e16)[0]
    idx, w16, w32 = o.router_select(logits, g16, 8)
    # the reference's own CPU reference: dequant-then-dot on (hidden * effectiveScale) in fp32, sort, softmax
    scaled = (o.f16_to_f32(h16) * o.bf16_to_f32(e16)).astype(np.float32)
    ref_logits = o.gemv_ref(mat, scaled)
    ridx, rw = o.router_select_sorted(ref_logits, o.bf16_to_f32(g16), 8)
    assert idx[0].tolist() == ridx.tolist()
    assert np.max(np.abs(o.f16_to_f32(w16[0]) - rw)) < 5e-3
    assert np.max(np.abs(logits - o.router_logits_f64(mat, h16, e16)[0])) < 1e-5


def test_router_near_tie(oracle):
    # RouterTopKTests.swift:47-70: gains 0.5 vs 0.5*(1+1e-4) on a positive pattern
    o = oracle
    rng = o.SplitMix64(0x71E0F4A)
    pattern = rng.uniform_array(0.2, 1.0, 128)
    hidden = rng.uniform_array(0.5, 1.5, 128)
    gains = np.zeros(16, dtype=np.float32)
    for e in range(7):
        gains[e] = np.float32(1.0) - np.float32(e) * np.float32(0.05)
    gains[7] = 0.5
    gains[8] = np.float32(0.5) * (np.float32(1.0) + np.float32(1e-4))
    for e in range(9, 16):
        gains[e] = np.float32(0.4) - np.float32(e - 9) * np.float32(0.02)
    weights = np.stack([pattern * g for g in gains])
    mat = o.quantize_rows(weights, 8)
    ones_bf = o.f32_to_bf16(np.ones(128, dtype=np.float32))
    h16 = o.f32_to_f16(hidden)
    logits = o.router_logits(mat, h16, ones_bf)[0]
    idx, _, _ = o.router_select(logits, o.f32_to_bf16(np.ones(16, dtype=np.float32)), 8)
    ridx, _ = o.router_select_sorted(o.gemv_ref(mat, o.f16_to_f32(h16)), np.ones(16, dtype=np.float32), 8)
    assert idx[0].tolist() == ridx.tolist()
    assert idx[0, :7].tolist() == list(range(7)) and int(idx[0, 7]) in (7, 8)


def test_topk_ties_go_to_lower_index(oracle):
    logits = np.array([1.0, 3.0, 3.0, 2.0, 3.0, 0.5, 2.0, 2.0, 2.0, 2.0, -1.0, 2.0], dtype=np.float32)
    idx, _, w = oracle.router_select(logits, oracle.f32_to_bf16(np.ones(12, dtype=np.float32)), 8)
    assert idx[0].tolist() == [1, 2, 4, 3, 6, 7, 8, 9]
    assert abs(float(w[0].sum()) - 1.0) < 1e-6


def test_moe_routed_kernel_order_vs_truth(oracle):
    # MoEFusedFFNTests.swift:17-159: D=128, F=64, K=8, seed 0x2D3, weights 0.04+0.015k; rel < 1e-2
    o = oracle
    D, F, K = 128, 64, 8
    rng = o.SeedTree(0x2D3).key("production-routed-moe")
    off, payload, stride = o.blob_layout(D, F, align=256)
    blobs = []
    for _ in range(K):
        gate = o.quantize_rows(np.stack([rng.uniform_array(-0.5, 0.5, D) for _ in range(F)]), 4)
        up = o.quantize_rows(np.stack([rng.uniform_array(-0.5, 0.5, D) for _ in range(F)]), 4)
        down = o.quantize_rows(np.stack([rng.uniform_array(-0.5, 0.5, F) for _ in range(D)]), 4)
        blobs.append(o.pack_blob(gate, up, down, off, stride))
    x16 = o.f32_to_f16(rng.uniform_array(-1.0, 1.0, D))
    w16 = o.f32_to_f16(np.array([0.04 + 0.015 * k for k in range(K)], dtype=np.float32))
    res = o.f32_to_f16(np.zeros(D, dtype=np.float32))
    y_truth16, y_truth, _ = o.moe_routed_decode(blobs, off, x16, w16, res, D, F, order=0)
    y_k16, y_k, _ = o.moe_routed_decode(blobs, off, x16, w16, res, D, F, order=1)
    assert o.rel_error(o.f16_to_f32(y_k16), y_truth) < 1e-2
    assert o.rel_error(y_k, y_truth) < 2e-3


def test_reduce_token_major_matches_numpy(oracle):
    # PrefillMoETests.swift:8-64 (seed 0x4D0E2026, 3 x 8 x 64; max-abs <= 2e-3)
    o = oracle
    rng = o.SplitMix64(0x4D0E2026)
    T, K, D = 3, 8, 64
    partials = o.f32_to_f16(rng.uniform_array(-1.0, 1.0, T * K * D).reshape(T, K, D))
    weights = o.f32_to_f16(rng.uniform_array(0.0, 0.25, T * K).reshape(T, K))
    out = o.f16_to_f32(o.moe_reduce_token_major(partials, weights, T, K, D))
    ref = np.einsum("tk,tkd->td", o.f16_to_f32(weights).astype(np.float64), o.f16_to_f32(partials).astype(np.float64))
    assert np.max(np.abs(out - ref)) <= 2e-3


def test_rmsnorm_and_tail_against_float64(oracle):
    o = oracle
    rng = np.random.default_rng(11)
    D = 2816
    x = o.f32_to_f16(rng.standard_normal((3, D)).astype(np.float32))
    w = o.f32_to_bf16((1 + 0.02 * rng.standard_normal(D)).astype(np.float32))
    y = o.f16_to_f32(o.rmsnorm(x, w))
    xf = o.f16_to_f32(x).astype(np.float64)
    ref = xf / np.sqrt((xf ** 2).mean(axis=1, keepdims=True) + 1e-6) * o.bf16_to_f32(w)
    assert o.rel_error(y, ref) < 1e-3
    y0 = o.f16_to_f32(o.rmsnorm(x, None))
    assert o.rel_error(y0, xf / np.sqrt((xf ** 2).mean(axis=1, keepdims=True) + 1e-6)) < 1e-3
    h2, h1, hid = x, o.f32_to_f16(rng.standard_normal((3, D)).astype(np.float32)), o.f32_to_f16(rng.standard_normal((3, D)).astype(np.float32))
    out = o.f16_to_f32(o.layer_tail(h2, h1, hid, w, w, layer_scalar=0.5))
    n = lambda a: a / np.sqrt((a ** 2).mean(axis=1, keepdims=True) + 1e-6)
    wf = o.bf16_to_f32(w).astype(np.float64)
    ref = (o.f16_to_f32(hid) + n(o.f16_to_f32(h1) + n(xf) * wf) * wf) * 0.5
    assert o.rel_error(out, ref) < 5e-3
