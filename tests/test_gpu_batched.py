"""GPU parity of the batched (multi-token) routed-expert path: device grouping, grouped
gate/up + down kernels, token-major reduce and the batched shared expert."""
import numpy as np
import pytest

from helpers import capi_offsets, config0_matrix, dev_zeros_u16, from_dev, random_blob, to_dev

pytestmark = pytest.mark.gpu
FP16_CHAINED = 1e-2


def _route(rng, T, K, E, zipf=False):
    if zipf:
        p = 1.0 / (rng.permutation(E) + 1) ** 1.1
        p /= p.sum()
        idx = np.stack([rng.choice(E, size=K, replace=False, p=p) for _ in range(T)])
    else:
        idx = np.stack([rng.permutation(E)[:K] for _ in range(T)])
    return idx.astype(np.uint32)


@pytest.mark.parametrize("T,K,E,zipf", [(1, 8, 128, False), (64, 8, 128, False), (300, 8, 128, True), (4096, 8, 128, True),
                                         (3, 2, 16, False), (7, 3, 5, False),
                                         # from 4096 pairs on: slices of pairs, three launches (ragged last slice, E not a multiple of 32)
                                         (513, 8, 128, False), (700, 8, 250, True), (20000, 8, 128, True)])
def test_device_grouping_matches_oracle(tf_ctx, oracle, T, K, E, zipf):
    import torch
    from turbo_fieldfare_b200.kernels import DeviceRoutes, PrefillGroupedRoutedMoE
    o = oracle
    rng = np.random.default_rng(T * 7 + K)
    idx = _route(rng, T, K, E, zipf)
    if T >= 64:
        idx[5, 3] = E + 9            # out-of-range id clamps to E-1 (RealForwardRunner.swift:955)
    w16 = rng.integers(0, 0x3C00, size=(T, K)).astype(np.uint16)
    routes = DeviceRoutes(T, K, E)
    PrefillGroupedRoutedMoE(tf_ctx).encode_group_routes(to_dev(idx), to_dev(w16), T, K, E, routes)
    torch.cuda.synchronize()
    got = routes.to_host(T)
    ref = o.group_pairs(o.make_token_expert_pairs(np.minimum(idx, E - 1), w16, T, K), T, K, E, 16)
    assert got.sorted_pairs.tobytes() == ref.sorted_pairs.tobytes()
    assert np.array_equal(got.per_expert_offsets, ref.per_expert_offsets)
    assert np.array_equal(got.per_expert_counts, ref.per_expert_counts)
    assert got.groups.tobytes() == ref.groups.tobytes()
    counters = routes.counters.cpu().numpy().view(np.uint32)
    assert counters[0] == len(ref.groups) and counters[2] == T * K and counters[3] == T * K
    assert counters[1] == sum((int(c) + 7) // 8 for c in ref.per_expert_counts)


def _closed_form_pool(o, E, D, F):
    """Closed-form weights of the reference's grouped-MoE test
    (Tests/TurboFieldfare/Core/Kernels/Prefill/PrefillGroupedRoutedMoETests.swift:114-216)."""
    off, payload, stride = o.blob_layout(D, F, align=256)
    pool = np.zeros(E * stride, dtype=np.uint8)
    for e in range(E):
        mats = []
        for role, (rows, cols) in enumerate(((F, D), (F, D), (D, F))):
            r = np.arange(rows)[:, None]
            c = np.arange(cols)[None, :]
            w = (e + 1) * 0.001 + (role + 1) * 0.003 + ((r % 7) - 3) * 0.0004 + ((c % 11) - 5) * 0.0002
            mats.append(o.quantize_rows(w.astype(np.float32), 4))
        pool[e * stride:(e + 1) * stride] = o.pack_blob(*mats, off, stride)
    return pool, off, stride


def _run_batched(tf_ctx, o, pool_h, off, stride, hidden16, idx, w16, D, F, K, E, partials_f32=False):
    import torch
    from turbo_fieldfare_b200.kernels import DeviceRoutes, PrefillGroupedRoutedMoE
    T = hidden16.shape[0]
    routes = DeviceRoutes(T, K, E)
    moe = PrefillGroupedRoutedMoE(tf_ctx)
    moe.encode_group_routes(to_dev(idx), to_dev(w16), T, K, E, routes)
    pool = to_dev(pool_h)
    acts = dev_zeros_u16(T * K * F)
    if partials_f32:
        partials = torch.full((T * K * D,), float("nan"), dtype=torch.float32, device="cuda")
    else:
        partials = dev_zeros_u16(T * K * D, fill=0x7E00)
    moe.encode_streamed_batched(to_dev(hidden16), pool, stride, capi_offsets(off), routes, acts, partials, T, D, F, K,
                                partials_f32=partials_f32)
    torch.cuda.synchronize()
    assert tf_ctx.device_status() == 0, "a kernel abandoned a bounded wait"
    if partials_f32:
        return partials.cpu().numpy().reshape(T, K, D), routes
    return from_dev(partials, np.uint16).reshape(T, K, D), routes


def test_grouped_moe_closed_form_fixture(tf_ctx, oracle):
    # 16 experts, D=F=64, 3 tokens x top-2, hidden ((i % 17) - 8) * 0.01; max-abs <= 0.0015
    o = oracle
    E, D, F, T, K = 16, 64, 64, 3, 2
    pool, off, stride = _closed_form_pool(o, E, D, F)
    hidden = (((np.arange(T * D) % 17) - 8) * 0.01).astype(np.float32).reshape(T, D)
    h16 = o.f32_to_f16(hidden)
    idx = np.array([[3, 9], [9, 1], [15, 3]], dtype=np.uint32)
    w16 = o.f32_to_f16(np.full((T, K), 0.5, dtype=np.float32))
    got, _ = _run_batched(tf_ctx, o, pool, off, stride, h16, idx, w16, D, F, K, E)
    pairs = o.make_token_expert_pairs(idx, w16, T, K)
    ref = o.grouped_moe_pairs(pool, stride, off, h16, 0, pairs, D, F, K, T)
    assert np.max(np.abs(o.f16_to_f32(got) - o.f16_to_f32(ref))) <= 0.0015


def _run_streamed(tf_ctx, o, blobs_h, bound_experts, off, hidden16, pairs_sorted, pair_start, pair_count, D, F, K, microbatch=4):
    """tf_grouped_moe_streamed on separately allocated blobs (one device buffer per bound expert, in the given slot order)."""
    import ctypes as C
    import torch
    from turbo_fieldfare_b200._capi import StreamedParams
    from turbo_fieldfare_b200.kernels import _ptr
    T = hidden16.shape[0]
    devs = [to_dev(b) for b in blobs_h]
    table = (C.c_void_p * len(devs))(*[d.data_ptr() for d in devs])
    p = StreamedParams()
    p.pair_start, p.pair_count, p.d, p.routed_intermediate, p.top_k, p.hidden_stride_elements = pair_start, pair_count, D, F, K, D
    p.live_expert_count = len(devs)
    for i in range(16):
        p.local_expert[i] = bound_experts[i] if i < len(bound_experts) else 0xFFFFFFFF
    (p.gate_w_off, p.gate_s_off, p.gate_b_off, p.up_w_off, p.up_s_off, p.up_b_off, p.down_w_off, p.down_s_off, p.down_b_off) = (
        off.gate_w, off.gate_s, off.gate_b, off.up_w, off.up_s, off.up_b, off.down_w, off.down_s, off.down_b)
    pairs_dev = to_dev(np.ascontiguousarray(pairs_sorted).view(np.uint32))
    partials = dev_zeros_u16(T * K * D, fill=0x7E00)
    acts = dev_zeros_u16(max(pair_count, 1) * F)
    n_mb = C.c_uint32(99)
    tf_ctx.check(tf_ctx.lib.tf_grouped_moe_streamed(tf_ctx.handle, 0, _ptr(to_dev(hidden16)), 0, _ptr(pairs_dev), 0, _ptr(partials), 0,
                                                    _ptr(acts), 0, table, len(devs), C.byref(p), microbatch, C.byref(n_mb)))
    torch.cuda.synchronize()
    return from_dev(partials, np.uint16).reshape(T, K, D), int(n_mb.value)


def test_grouped_moe_streamed_closed_form_fixture(tf_ctx, oracle):
    """The reference's streamed execution test (PrefillGroupedRoutedMoETests+Execution.swift:8-103): the closed-form
    fixture through the tile-binding form (blob addresses + the 128-byte parameter block), max-abs <= 0.0015, two
    microbatches at four rows; bound experts in an order that is not the sorted one; then only part of the pairs."""
    o = oracle
    E, D, F, T, K = 16, 64, 64, 3, 2
    pool, off, stride = _closed_form_pool(o, E, D, F)
    hidden = (((np.arange(T * D) % 17) - 8) * 0.01).astype(np.float32).reshape(T, D)
    h16 = o.f32_to_f16(hidden)
    idx = np.array([[3, 9], [9, 1], [15, 3]], dtype=np.uint32)
    w16 = o.f32_to_f16(np.full((T, K), 0.5, dtype=np.float32))
    pairs = o.make_token_expert_pairs(idx, w16, T, K)
    routes = o.group_pairs(pairs, T, K, E)
    sorted_pairs = routes.sorted_pairs
    ref = o.f16_to_f32(o.grouped_moe_pairs(pool, stride, off, h16, 0, pairs, D, F, K, T))
    bound = [9, 1, 15, 3]                                  # slot order differs from the sorted expert order
    blobs = [pool[e * stride:(e + 1) * stride].copy() for e in bound]
    got, n_mb = _run_streamed(tf_ctx, o, blobs, bound, off, h16, sorted_pairs, 0, T * K, D, F, K, microbatch=4)
    assert tf_ctx.device_status() == 0
    assert n_mb == 2
    assert np.max(np.abs(o.f16_to_f32(got) - ref)) <= 0.0015
    # the second half of the sorted pairs only: the other partial rows stay untouched
    got2, n_mb2 = _run_streamed(tf_ctx, o, blobs, bound, off, h16, sorted_pairs, 3, 3, D, F, K, microbatch=32)
    assert n_mb2 == 1 and tf_ctx.device_status() == 0
    touched = np.zeros((T, K), dtype=bool)
    for pr in sorted_pairs[3:6]:
        touched[int(pr["token"]), int(pr["rank"])] = True
    assert np.max(np.abs(o.f16_to_f32(got2)[touched] - ref[touched])) <= 0.0015
    assert (got2[~touched] == 0x7E00).all()
    # nothing to do (PrefillGroupedRoutedMoE.swift:402-404): no launch, zero microbatches
    before = tf_ctx.launch_count
    _, n0 = _run_streamed(tf_ctx, o, blobs, bound, off, h16, sorted_pairs, 0, 0, D, F, K)
    assert n0 == 0 and tf_ctx.launch_count == before


def test_grouped_moe_streamed_reports_unbound_expert(tf_ctx, oracle):
    """A pair whose expert is not bound in the tile is skipped and reported (the reference validates this on the
    host: PrefillStreamedTileBinding.validateCoversPairs, PrefillGroupedRoutedMoE.swift:287-301)."""
    from turbo_fieldfare_b200.kernels import TFError
    o = oracle
    E, D, F, T, K = 16, 64, 64, 3, 2
    pool, off, stride = _closed_form_pool(o, E, D, F)
    h16 = o.f32_to_f16((((np.arange(T * D) % 17) - 8) * 0.01).astype(np.float32).reshape(T, D))
    idx = np.array([[3, 9], [9, 1], [15, 3]], dtype=np.uint32)
    w16 = o.f32_to_f16(np.full((T, K), 0.5, dtype=np.float32))
    pairs = o.make_token_expert_pairs(idx, w16, T, K)
    sorted_pairs = o.group_pairs(pairs, T, K, E).sorted_pairs
    bound = [1, 3, 9]                                       # expert 15 is missing
    blobs = [pool[e * stride:(e + 1) * stride].copy() for e in bound]
    got, _ = _run_streamed(tf_ctx, o, blobs, bound, off, h16, sorted_pairs, 0, T * K, D, F, K)
    with pytest.raises(TFError):
        tf_ctx.device_status()
    assert tf_ctx.device_status() == 0                      # reported once, then cleared
    ref = o.f16_to_f32(o.grouped_moe_pairs(pool, stride, off, h16, 0, pairs, D, F, K, T))
    ok = idx != 15
    assert np.max(np.abs(o.f16_to_f32(got)[ok] - ref[ok])) <= 0.0015
    assert (got[~ok] == 0x7E00).all()


@pytest.mark.parametrize("T,D,F,E,K", [(1, 128, 64, 16, 8), (5, 128, 64, 16, 8), (40, 256, 128, 8, 4), (64, 2816, 704, 16, 8)])
def test_grouped_moe_random_vs_oracle(tf_ctx, oracle, T, D, F, E, K):
    """Config-2 style: T tokens scattered over E experts (up to 64 x 8 pairs on 16 experts: chunks of 8 and ragged tails)."""
    o = oracle
    rng = np.random.default_rng(T + D)
    off, payload, stride = o.blob_layout(D, F, align=256 if D < 2816 else 16384)
    pool = np.zeros(E * stride, dtype=np.uint8)
    for e in range(E):
        pool[e * stride:(e + 1) * stride] = random_blob(o, D, F, rng, off, stride)[0]
    h16 = o.f32_to_f16(rng.standard_normal((T, D)).astype(np.float32))
    idx = _route(rng, T, K, E)
    w16 = o.f32_to_f16(rng.dirichlet(np.ones(K), size=T).astype(np.float32))
    pairs = o.make_token_expert_pairs(idx, w16, T, K)
    ref = o.f16_to_f32(o.grouped_moe_pairs(pool, stride, off, h16, 0, pairs, D, F, K, T))
    got16, _ = _run_batched(tf_ctx, o, pool, off, stride, h16, idx, w16, D, F, K, E)
    got = o.f16_to_f32(got16)
    assert o.rel_l2(got, ref) < FP16_CHAINED
    assert o.rel_error(got, ref) < FP16_CHAINED
    got32, _ = _run_batched(tf_ctx, o, pool, off, stride, h16, idx, w16, D, F, K, E, partials_f32=True)
    assert o.rel_l2(got32, ref) < FP16_CHAINED
    # batched path == decode path per token within tolerance (the reference checks block == repeated decode)
    if T <= 5:
        for t in range(T):
            blobs = [pool[int(e) * stride:(int(e) + 1) * stride] for e in idx[t]]
            _, y32, _ = o.moe_routed_decode(blobs, off, h16[t], w16[t], None, D, F, order=0)
            y_batched = (o.f16_to_f32(w16[t])[:, None] * got32[t]).sum(axis=0)
            assert o.rel_error(y_batched, y32) < FP16_CHAINED


def test_reduce_token_major(tf_ctx, oracle):
    # Tests/TurboFieldfare/Core/Kernels/Prefill/PrefillMoETests.swift:8-64
    import torch
    from turbo_fieldfare_b200.kernels import PrefillMoE
    o = oracle
    rng = o.SplitMix64(0x4D0E2026)
    T, K, D = 3, 8, 64
    partials = o.f32_to_f16(rng.uniform_array(-1.0, 1.0, T * K * D).reshape(T, K, D))
    weights = o.f32_to_f16(rng.uniform_array(0.0, 0.25, T * K).reshape(T, K))
    h2 = dev_zeros_u16(T * D)
    PrefillMoE(tf_ctx).encode_reduce_token_major(to_dev(partials), to_dev(weights), h2, T, K, D)
    torch.cuda.synchronize()
    ref = o.moe_reduce_token_major(partials, weights, T, K, D)
    assert from_dev(h2, np.uint16).tobytes() == ref.tobytes()      # same fma chain: bit-exact


@pytest.mark.parametrize("T", [1, 3, 17, 64])
def test_shared_expert_block_vs_rows(tf_ctx, oracle, T):
    """Block shared expert == per-row shared expert (PrefillSharedExpertTests.swift:89,177,243 checks equality)."""
    import torch
    from turbo_fieldfare_b200.kernels import PrefillSharedExpert, SharedExpertProjection
    o = oracle
    rng = np.random.default_rng(1234 + T)
    D, Fs = (2816, 2112) if T in (1, 64) else (128, 192)
    gate, up, down = config0_matrix(o, Fs, D, rng), config0_matrix(o, Fs, D, rng), config0_matrix(o, D, Fs, rng)
    x16 = o.f32_to_f16(rng.standard_normal((T, D)).astype(np.float32))
    proj = lambda m: SharedExpertProjection(to_dev(m.packed), to_dev(m.scales), to_dev(m.biases), m.m, m.n)
    y = dev_zeros_u16(T * D)
    scratch = dev_zeros_u16(T * Fs)
    PrefillSharedExpert(tf_ctx).encode_block(to_dev(x16), proj(gate), proj(up), proj(down), y, scratch, T)
    torch.cuda.synchronize()
    got = o.f16_to_f32(from_dev(y, np.uint16).reshape(T, D))
    rows = range(T) if T <= 17 else (0, 31, 63)
    for t in rows:
        _, truth = o.shared_expert_int4(gate, up, down, x16[t], order=0)
        assert o.rel_l2(got[t], truth) < FP16_CHAINED
        assert o.rel_error(got[t], truth) < FP16_CHAINED
