"""GPU parity of the decode-path entry points against the CPU oracle, through the
C ABI. Seeds, shapes and tolerances are the reference's own where it has a test
(cited per case); benchmark configurations use numpy-seeded inputs."""
import numpy as np
import pytest

from helpers import (blob_table, capi_offsets, config0_matrix, dev_zeros_u16, from_dev, quantized_blob, random_blob,
                     to_dev)

pytestmark = pytest.mark.gpu

FP16_REDUCTION = 5e-3      # Tolerance.fp16Reduction
FP16_CHAINED = 1e-2        # Tolerance.fp16ChainedReduction (also the benchmark's 1e-2 relative L2)


def _run_gemv(tf_ctx, o, mat, x16, offset=0, bits=4):
    import torch
    from turbo_fieldfare_b200.kernels import DequantInt4GEMV, DequantInt8GEMV
    raw = mat.packed.reshape(-1)
    padded = np.zeros(raw.size + offset + 16, dtype=np.uint8)
    padded[offset:offset + raw.size] = raw
    W, S, B, x = to_dev(padded), to_dev(mat.scales), to_dev(mat.biases), to_dev(x16)
    guard = 8
    y = dev_zeros_u16(mat.m + 2 * guard, fill=0x7BFF)        # poison: 65504
    k = (DequantInt4GEMV if bits == 4 else DequantInt8GEMV)(tf_ctx)
    k.encode(W, S, B, x, y, mat.m, mat.n, weights_offset=offset, y_offset=guard * 2, sb_dtype=mat.sb_dtype)
    torch.cuda.synchronize()
    out = from_dev(y, np.uint16)
    assert np.all(out[:guard] == 0x7BFF) and np.all(out[-guard:] == 0x7BFF), "guard band overwritten"
    return out[guard:-guard]


@pytest.mark.parametrize("m,n,seed,label,offset", [
    (128, 128, 0xC1, "int4-gemv-kernel-m128-n128", 0),
    (1024, 2816, 0xC2, "int4-gemv-kernel-m1024-n2816", 0),
    (64, 64, 0xC3, "int4-gemv-kernel-m64-n64", 0),
    (128, 2816, 0xC4, "int4-gemv-kernel-m128-n2816-off2", 2),
])
def test_int4_gemv_reference_fixtures(tf_ctx, oracle, m, n, seed, label, offset):
    # Tests/TurboFieldfare/Core/Kernels/Quant/DequantInt4GEMVTests.swift:41-121
    o = oracle
    rng = o.SeedTree(seed).key(label)
    mat = o.quantize_rows(np.stack([rng.uniform_array(-0.5, 0.5, n) for _ in range(m)]), 4)
    x16 = o.f32_to_f16(rng.uniform_array(-1.0, 1.0, n))
    y = _run_gemv(tf_ctx, o, mat, x16, offset)
    ref = o.gemv_ref(mat, o.f16_to_f32(x16))
    assert o.rel_error(o.f16_to_f32(y), ref) < FP16_REDUCTION
    assert o.rel_l2(o.f16_to_f32(y), ref) < 1e-3


@pytest.mark.parametrize("m", [64, 65, 128, 129])
@pytest.mark.parametrize("n", [64, 128, 192, 256, 320, 384, 448, 512])
def test_int4_gemv_sweep(tf_ctx, oracle, m, n):
    # DequantInt4GEMVTests.swift:123-128
    o = oracle
    seed = (m * 0x9E37 + n) & 0xFFFFFFFFFFFFFFFF
    rng = o.SeedTree(seed).key(f"int4-gemv-kernel-m{m}-n{n}")
    mat = o.quantize_rows(np.stack([rng.uniform_array(-0.5, 0.5, n) for _ in range(m)]), 4)
    x16 = o.f32_to_f16(rng.uniform_array(-1.0, 1.0, n))
    y = _run_gemv(tf_ctx, o, mat, x16)
    assert o.rel_error(o.f16_to_f32(y), o.gemv_ref(mat, o.f16_to_f32(x16))) < FP16_REDUCTION


@pytest.mark.parametrize("m,n,seed", [(128, 2816, 0x151), (1024, 2816, 0x152)])
def test_int8_gemv_reference_fixtures(tf_ctx, oracle, m, n, seed):
    # DequantInt8GEMVTests.swift:74-88
    o = oracle
    rng = o.SplitMix64(seed)
    mat = o.quantize_rows(np.stack([rng.uniform_array(-0.5, 0.5, n) for _ in range(m)]), 8)
    x16 = o.f32_to_f16(rng.uniform_array(-1.0, 1.0, n))
    for offset in (0, 1):
        y = _run_gemv(tf_ctx, o, mat, x16, offset=offset, bits=8)
        assert o.rel_error(o.f16_to_f32(y), o.gemv_ref(mat, o.f16_to_f32(x16))) < FP16_REDUCTION


@pytest.mark.parametrize("sb_dtype", [0, 1])
def test_config0_gemv_704x2816(tf_ctx, oracle, sb_dtype):
    """benchmark configuration 0: 704 x 2816, uniform codes, scale/bias distributions, x ~ N(0,1) fp16."""
    o = oracle
    rng = np.random.default_rng(20260 + sb_dtype)
    mat = config0_matrix(o, 704, 2816, rng, sb_dtype=sb_dtype)
    x16 = o.f32_to_f16(rng.standard_normal(2816).astype(np.float32))
    y = o.f16_to_f32(_run_gemv(tf_ctx, o, mat, x16))
    ref = o.gemv_ref(mat, o.f16_to_f32(x16))
    assert o.rel_l2(y, ref) < FP16_CHAINED
    assert o.rel_error(y, ref) < FP16_REDUCTION


def test_gemv_rejects_bad_arguments(tf_ctx, oracle):
    from turbo_fieldfare_b200.kernels import DequantInt4GEMV, TFError
    import torch
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    k = DequantInt4GEMV(tf_ctx)
    with pytest.raises(TFError) as e:
        k.encode(buf, buf, buf, buf, buf, 4, 96)          # N % 64 != 0 (DequantInt4GEMV.swift:57-62)
    assert e.value.status == 1
    with pytest.raises(TFError) as e:
        k.encode(buf, buf, buf, buf, buf, 4, 64, weights_offset=1)   # odd weights offset
    assert e.value.status == 4


# ---------------------------------------------------------------------------
# router
# ---------------------------------------------------------------------------

def _run_router(tf_ctx, o, mat, hidden16, eff16, gain16, rows=None, stride=None, logit_bias=None, bf16_hidden=False):
    import torch
    from turbo_fieldfare_b200.kernels import MoE, PrefillRouter
    E, D = mat.m, mat.n
    W, S, B = to_dev(mat.packed), to_dev(mat.scales), to_dev(mat.biases)
    eff, gain = to_dev(eff16), to_dev(gain16)
    hid = to_dev(hidden16)
    if rows is None:
        idx = torch.full((8,), -1, dtype=torch.int32, device="cuda")
        w = dev_zeros_u16(8)
        logits = torch.zeros(E, dtype=torch.float32, device="cuda")
        MoE(tf_ctx).encode_router_gemma4(W, S, B, hid, eff, gain, idx, w, E, D, 8, out_logits=logits)
        torch.cuda.synchronize()
        return from_dev(idx, np.uint32), from_dev(w, np.uint16), logits.cpu().numpy()
    K = 8
    idx = torch.full((rows, K), -1, dtype=torch.int32, device="cuda")
    w = dev_zeros_u16(rows * K)
    logits = torch.zeros((rows, E), dtype=torch.float32, device="cuda")
    PrefillRouter(tf_ctx).encode_gemma4_block(W, S, B, hid, eff, gain, idx, w, rows, E, D, K, stride or D,
                                              hidden_dtype=0 if bf16_hidden else 1,
                                              logit_bias=None if logit_bias is None else to_dev(logit_bias),
                                              out_logits=logits)
    torch.cuda.synchronize()
    return from_dev(idx, np.uint32).reshape(rows, K), from_dev(w, np.uint16).reshape(rows, K), logits.cpu().numpy()


@pytest.mark.parametrize("rows,E,D,skew", [(1, 128, 2816, 0.0), (5, 128, 2816, 0.0), (64, 128, 2816, 0.0),
                                           (64, 128, 2816, 6.0), (37, 16, 128, 0.0), (64, 256, 256, 2.0), (100, 128, 2816, 0.0),
                                           (1, 128, 2816, -np.inf), (3, 16, 128, -np.inf)])
def test_router_with_grouping_in_one_launch_equals_the_two_calls(tf_ctx, oracle, rows, E, D, skew):
    """Blocks of at most 64 rows route and group in one launch (the block that finishes the last row sorts the
    pairs); every routing table must equal what the router followed by the grouping launch writes, skewed loads
    (one expert taking most pairs) and the larger-block fallback included. Called twice to show the tickets reset."""
    import torch
    from turbo_fieldfare_b200.kernels import DeviceRoutes, PrefillGroupedRoutedMoE, PrefillRouter
    o = oracle
    K = 8
    rng = np.random.default_rng(rows * 1000 + E + D)
    mat = config0_matrix(o, E, D, rng, bits=8)
    hidden = o.f32_to_f16(rng.standard_normal((rows, D)).astype(np.float32))
    eff = o.f32_to_bf16(np.full(D, 1.0 / np.sqrt(D), np.float32))
    gain = o.f32_to_bf16(np.ones(E, np.float32))
    bias = None
    if skew == -np.inf:
        # only three experts stay selectable: the selection repeats expert 0 for the missing picks, and the grouping
        # has to merge the repeats into one group
        b = np.full(E, -np.inf, np.float32); b[[2, 5, E - 1]] = 0.0
        bias = to_dev(b)
    elif skew:
        b = np.zeros(E, np.float32); b[3] = skew; b[E - 1] = skew / 2
        bias = to_dev(b)
    W, S, B = to_dev(mat.packed), to_dev(mat.scales), to_dev(mat.biases)
    hid, effd, gaind = to_dev(hidden), to_dev(eff), to_dev(gain)
    launches = tf_ctx.launch_count

    def tables(routes, idx, w):
        torch.cuda.synchronize()
        n = rows * K
        counters = from_dev(routes.counters, np.uint32)
        ng, nch = int(counters[0]), int(counters[1])
        return dict(idx=from_dev(idx, np.uint32), w=from_dev(w, np.uint16),
                    pairs=from_dev(routes.sorted_pairs, np.uint32)[:n * 4], offsets=from_dev(routes.per_expert_offsets, np.uint32),
                    counts=from_dev(routes.per_expert_counts, np.uint32), groups=from_dev(routes.groups, np.uint32)[:ng * 3],
                    chunk_group=from_dev(routes.chunk_group, np.uint32)[:nch], chunk_start=from_dev(routes.chunk_start, np.uint32)[:ng],
                    counters=counters[:3])

    ref_routes = DeviceRoutes(rows, K, E)
    idx0 = torch.full((rows, K), -1, dtype=torch.int32, device="cuda"); w0 = dev_zeros_u16(rows * K)
    PrefillRouter(tf_ctx).encode_gemma4_block(W, S, B, hid, effd, gaind, idx0, w0, rows, E, D, K, D, logit_bias=bias)
    PrefillGroupedRoutedMoE(tf_ctx).encode_group_routes(idx0, w0, rows, K, E, ref_routes)
    want = tables(ref_routes, idx0, w0)
    assert want["counters"][2] == rows * K and want["counts"].sum() == rows * K
    if skew == -np.inf:
        assert want["counters"][0] == 4 and want["counts"][0] == rows * (K - 3)      # experts 0 (repeated), 2, 5, E - 1
    for attempt in range(2):
        routes = DeviceRoutes(rows, K, E)
        idx1 = torch.full((rows, K), -1, dtype=torch.int32, device="cuda"); w1 = dev_zeros_u16(rows * K)
        before = tf_ctx.launch_count
        PrefillRouter(tf_ctx).encode_gemma4_block_grouped(W, S, B, hid, effd, gaind, idx1, w1, rows, E, D, K, D, routes,
                                                          logit_bias=bias)
        assert tf_ctx.launch_count - before == (1 if rows <= 64 else 2)
        got = tables(routes, idx1, w1)
        for key in want:
            assert np.array_equal(got[key], want[key]), (key, attempt)
    assert tf_ctx.device_status() == 0 and tf_ctx.launch_count > launches


def test_router_reference_fixture(tf_ctx, oracle):
    # Tests/TurboFieldfare/Core/Kernels/MoE/RouterTopKTests.swift:17-45
    from test_oracle_pins import _router_fixture
    o = oracle
    weights, hidden, eff, gain = _router_fixture(o)
    mat = o.quantize_rows(weights, 8)
    h16, e16, g16 = o.f32_to_f16(hidden), o.f32_to_bf16(eff), o.f32_to_bf16(gain)
    idx, w16, logits = _run_router(tf_ctx, o, mat, h16, e16, g16)
    ref_logits = o.router_logits(mat, h16, e16)[0]
    assert logits.tobytes() == ref_logits.tobytes(), "router logits are not bit-exact with the canonical order"
    ridx, rw16, rw32 = o.router_select(ref_logits, g16, 8)
    assert idx.tolist() == ridx[0].tolist()
    assert np.max(np.abs(o.f16_to_f32(w16) - rw32[0])) < 5e-3
    # and against the reference test's own CPU formulation
    sidx, sw = o.router_select_sorted(o.gemv_ref(mat, (o.f16_to_f32(h16) * o.bf16_to_f32(e16)).astype(np.float32)),
                                      o.bf16_to_f32(g16), 8)
    assert idx.tolist() == sidx.tolist()
    assert np.max(np.abs(o.f16_to_f32(w16) - sw)) < 5e-3


def test_router_near_tie(tf_ctx, oracle):
    # RouterTopKTests.swift:47-70
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
    mat = o.quantize_rows(np.stack([pattern * g for g in gains]), 8)
    ones_d, ones_e = o.f32_to_bf16(np.ones(128, dtype=np.float32)), o.f32_to_bf16(np.ones(16, dtype=np.float32))
    h16 = o.f32_to_f16(hidden)
    idx, _, logits = _run_router(tf_ctx, o, mat, h16, ones_d, ones_e)
    ref_logits = o.router_logits(mat, h16, ones_d)[0]
    assert logits.tobytes() == ref_logits.tobytes()
    assert idx.tolist() == o.router_select(ref_logits, ones_e, 8)[0][0].tolist()
    assert idx.tolist() == o.router_select_sorted(o.gemv_ref(mat, o.f16_to_f32(h16)), np.ones(16, np.float32), 8)[0].tolist()


def test_router_exact_ties_lower_index_first(tf_ctx, oracle):
    """Identical rows give identical logits: the selection must take the lower ids."""
    o = oracle
    rng = np.random.default_rng(5)
    row = rng.uniform(-0.05, 0.05, 128).astype(np.float32)
    weights = np.stack([row] * 12 + [row * 0.5] * 4)
    mat = o.quantize_rows(weights, 8)
    h16 = o.f32_to_f16(rng.uniform(0.5, 1.0, 128).astype(np.float32) * np.sign(row))
    ones_d, ones_e = o.f32_to_bf16(np.ones(128, dtype=np.float32)), o.f32_to_bf16(np.ones(16, dtype=np.float32))
    idx, w16, _ = _run_router(tf_ctx, o, mat, h16, ones_d, ones_e)
    assert idx.tolist() == list(range(8))
    assert np.allclose(o.f16_to_f32(w16), 0.125, atol=1e-3)


@pytest.mark.parametrize("rows", [5, 64, 200, 259, 1024])     # from 256 rows: the eight-rows-per-block kernel (ragged last block at 259)
def test_block_router_strided_rows(tf_ctx, oracle, rows):
    # Tests/TurboFieldfare/Core/Kernels/Prefill/PrefillRouterTests.swift:33-101: stride D+13, sentinel padding
    o = oracle
    E, D, stride = 16, 128, 128 + 13
    rng = o.SplitMix64(0x9A7E2026)
    mat = o.quantize_rows(np.stack([rng.uniform_array(-0.05, 0.05, D) + np.float32(e) * np.float32(0.01) for e in range(E)]), 8)
    hidden = np.full((rows, stride), -31.0, dtype=np.float32)
    for t in range(rows):
        hidden[t, :D] = rng.uniform_array(-1.0, 1.0, D)
    h16 = o.f32_to_f16(hidden)
    e16 = o.f32_to_bf16(rng.uniform_array(0.5, 1.5, D) / np.sqrt(np.float32(D)))
    g16 = o.f32_to_bf16(rng.uniform_array(0.6, 1.4, E))
    idx, w16, logits = _run_router(tf_ctx, o, mat, h16, e16, g16, rows=rows, stride=stride)
    ref_logits = o.router_logits(mat, h16, e16, stride=stride)
    assert logits.tobytes() == ref_logits.tobytes()
    ridx, rw16, rw32 = o.router_select(ref_logits, g16, 8)
    assert np.array_equal(idx, ridx)
    assert np.max(np.abs(o.f16_to_f32(w16) - rw32)) < 5e-3


def test_production_router_128x2816_with_bias(tf_ctx, oracle):
    """benchmark configurations 1-3: 128 experts, D=2816, top-8; Zipf(1.1) logit bias; fp16 and bf16 rows."""
    o = oracle
    rng = np.random.default_rng(31)
    E, D, T = 128, 2816, 96
    mat = config0_matrix(o, E, D, rng, bits=8)
    eff = o.f32_to_bf16(np.full(D, 1.0 / np.sqrt(D), dtype=np.float32))
    gain = o.f32_to_bf16(np.ones(E, dtype=np.float32))
    ranks = rng.permutation(E) + 1
    p = 1.0 / ranks ** 1.1
    bias = np.log(p / p.sum()).astype(np.float32)
    x = rng.standard_normal((T, D)).astype(np.float32)
    for bf in (False, True):
        h16 = o.f32_to_bf16(x) if bf else o.f32_to_f16(x)
        idx, w16, logits = _run_router(tf_ctx, o, mat, h16, eff, gain, rows=T, logit_bias=bias, bf16_hidden=bf)
        if bf:
            # the oracle's logits take fp16 rows; for bf16 rows compare with the double-precision truth instead
            xf = o.bf16_to_f32(h16).astype(np.float64) * o.bf16_to_f32(eff).astype(np.float64)
            truth = xf @ o.dequantize(mat).astype(np.float64).T + bias
            assert np.max(np.abs(logits - truth)) < 1e-4
            order = np.argsort(-logits, axis=1, kind="stable")[:, :8]
            assert np.array_equal(idx, order.astype(np.uint32))
            continue
        ref_logits = (o.router_logits(mat, h16, eff) + bias).astype(np.float32)
        assert logits.tobytes() == ref_logits.tobytes()
        ridx, _, rw32 = o.router_select(ref_logits, gain, 8)
        assert np.array_equal(idx, ridx)
        assert np.max(np.abs(o.f16_to_f32(w16) - rw32)) < 5e-3
        # decode entry point on row 0 gives the same bits as the block entry point
        idx1, w1, lg1 = _run_router(tf_ctx, o, mat, h16[0], eff, gain)
        assert lg1.tobytes() == o.router_logits(mat, h16[0], eff)[0].tobytes()


@pytest.mark.parametrize("T", [2, 7, 33, 64])
def test_few_row_router_is_bit_exact(tf_ctx, oracle, T):
    """2 to 64 aligned rows take the kernel that computes a block of rows per expert pass: logits bit for bit those of the
    oracle's canonical order, indices equal, ragged last group of rows (7, 33) included; bf16 rows against the truth."""
    o = oracle
    rng = np.random.default_rng(7000 + T)
    E, D = 128, 2816
    mat = config0_matrix(o, E, D, rng, bits=8)
    eff = o.f32_to_bf16((rng.uniform(0.5, 1.5, D) / np.sqrt(D)).astype(np.float32))
    gain = o.f32_to_bf16(rng.uniform(0.6, 1.4, E).astype(np.float32))
    bias = (0.3 * rng.standard_normal(E)).astype(np.float32)
    x = rng.standard_normal((T, D)).astype(np.float32)
    h16 = o.f32_to_f16(x)
    idx, w16, logits = _run_router(tf_ctx, o, mat, h16, eff, gain, rows=T, logit_bias=bias)
    ref_logits = (o.router_logits(mat, h16, eff) + bias).astype(np.float32)
    assert logits.tobytes() == ref_logits.tobytes()
    ridx, _, rw32 = o.router_select(ref_logits, gain, 8)
    assert np.array_equal(idx, ridx)
    assert np.max(np.abs(o.f16_to_f32(w16) - rw32)) < 5e-3
    hb = o.f32_to_bf16(x)
    idx_b, _, logits_b = _run_router(tf_ctx, o, mat, hb, eff, gain, rows=T, logit_bias=bias, bf16_hidden=True)
    xf = o.bf16_to_f32(hb).astype(np.float64) * o.bf16_to_f32(eff).astype(np.float64)
    truth = xf @ o.dequantize(mat).astype(np.float64).T + bias
    assert np.max(np.abs(logits_b - truth)) < 1e-4
    assert np.array_equal(idx_b, np.argsort(-logits_b, axis=1, kind="stable")[:, :8].astype(np.uint32))
    assert tf_ctx.device_status() == 0


@pytest.mark.parametrize("rows,E,D,case,bf16", [(300, 16, 256, "plain", False), (1000, 128, 2816, "bias", False),
                                                (257, 250, 512, "few_finite", False), (700, 128, 2816, "some_ninf", True),
                                                (4096, 128, 2816, "twins", False), (513, 128, 2816, "odd_rows", False)])
def test_two_launch_router_equals_the_canonical_router(tf_ctx, oracle, rows, E, D, case, bf16):
    """Batches of 256 rows and more compute all logits on the tensor cores and re-check the experts that can reach the
    top 8 in the canonical order: indices and weights must be those of the one-launch kernel byte for byte (a call that
    asks for the logits takes the one-launch kernel, whose logits are checked against the oracle at full size).
    Cases: a logit bias; fewer than 8 experts with a finite bias; most experts at -inf; two experts with identical
    rows (an exact tie in every token); rows of zeros, subnormal, huge, infinite and NaN activations."""
    import torch
    from turbo_fieldfare_b200.kernels import PrefillRouter
    o = oracle
    rng = np.random.default_rng(9100 + rows + E)
    mat = config0_matrix(o, E, D, rng, bits=8)
    if case == "twins":
        for arr in (mat.packed, mat.scales, mat.biases):
            arr[77] = arr[3]
            arr[12] = arr[100]
    eff = o.f32_to_bf16((rng.uniform(0.5, 1.5, D) / np.sqrt(D)).astype(np.float32))
    gain = o.f32_to_bf16(rng.uniform(0.6, 1.4, E).astype(np.float32))
    bias = None
    if case == "bias":
        bias = (0.3 * rng.standard_normal(E)).astype(np.float32)
    elif case == "few_finite":
        bias = np.full(E, -np.inf, np.float32); bias[[2, 5, 100, E - 1]] = [0.0, 0.1, -0.2, 0.05]
    elif case == "some_ninf":
        bias = np.full(E, -np.inf, np.float32); bias[rng.permutation(E)[:20]] = 0.0
    x = rng.standard_normal((rows, D)).astype(np.float32)
    if case == "odd_rows":
        x[0] = 0.0
        x[1] = 1e-7                                   # subnormal in fp16
        x[2] *= 3000.0                                # the fp16 split of x * 2^10 overflows
        x[3, 17] = np.inf
        x[4, 5] = np.nan
        x[5] = 60000.0 * np.sign(x[5])
        x[6, :64] = 0.0
        x[7] *= 1e-3
    h = o.f32_to_bf16(x) if bf16 else o.f32_to_f16(x)
    W, S, B = to_dev(mat.packed), to_dev(mat.scales), to_dev(mat.biases)
    effd, gaind, hid = to_dev(eff), to_dev(gain), to_dev(h)
    biasd = None if bias is None else to_dev(bias)
    K = 8

    def run(want_logits, min_rows):
        tf_ctx.set_router_tensorcore_min_rows(min_rows)
        idx = torch.full((rows, K), -1, dtype=torch.int32, device="cuda")
        w = dev_zeros_u16(rows * K)
        logits = torch.zeros((rows, E), dtype=torch.float32, device="cuda") if want_logits else None
        PrefillRouter(tf_ctx).encode_gemma4_block(W, S, B, hid, effd, gaind, idx, w, rows, E, D, K, D,
                                                  hidden_dtype=0 if bf16 else 1, logit_bias=biasd, out_logits=logits)
        torch.cuda.synchronize()
        return from_dev(idx, np.uint32).reshape(rows, K), from_dev(w, np.uint16).reshape(rows, K)

    try:
        idx_one, w_one = run(False, 0xFFFFFFFF)         # the one-launch kernel
        idx_log, w_log = run(True, 256)                 # asks for the logits: the one-launch kernel as well
        idx_two, w_two = run(False, 256)                # tensor-core logits + canonical re-check
    finally:
        tf_ctx.set_router_tensorcore_min_rows(256)
    assert np.array_equal(idx_one, idx_log) and w_one.tobytes() == w_log.tobytes()
    bad = np.nonzero(np.any(idx_two != idx_one, axis=1))[0]
    assert bad.size == 0, f"rows {bad[:8]} differ: {idx_two[bad[:2]]} vs {idx_one[bad[:2]]}"
    assert w_two.tobytes() == w_one.tobytes()
    assert tf_ctx.device_status() == 0


def test_router_preconditions(tf_ctx):
    import torch
    from turbo_fieldfare_b200.kernels import MoE, TFError
    b = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    moe = MoE(tf_ctx)
    for kwargs in (dict(num_experts=16, d=100, top_k=8), dict(num_experts=300, d=128, top_k=8),
                   dict(num_experts=16, d=128, top_k=4)):          # MoE.swift:121-123
        with pytest.raises(TFError) as e:
            moe.encode_router_gemma4(b, b, b, b, b, b, b, b, **kwargs)
        assert e.value.status == 1


# ---------------------------------------------------------------------------
# routed experts, decode
# ---------------------------------------------------------------------------

def _routed_fixture(o, D=128, F=64, K=8):
    # Tests/TurboFieldfare/Core/Kernels/MoE/MoEFusedFFNTests.swift:17-159
    rng = o.SeedTree(0x2D3).key("production-routed-moe")
    off, payload, stride = o.blob_layout(D, F, align=256)
    blobs = [quantized_blob(o, D, F, rng.uniform_array, off, stride)[0] for _ in range(K)]
    x16 = o.f32_to_f16(rng.uniform_array(-1.0, 1.0, D))
    w16 = o.f32_to_f16(np.array([0.04 + 0.015 * k for k in range(K)], dtype=np.float32))
    return off, blobs, x16, w16


def test_routed_decode_reference_fixture(tf_ctx, oracle):
    import torch
    from turbo_fieldfare_b200.kernels import MoE
    o = oracle
    D, F, K = 128, 64, 8
    off, blobs, x16, w16 = _routed_fixture(o, D, F, K)
    # poison prefix/suffix around every blob (PrefillGroupedRoutedMoETests.swift:80-106 style)
    dev_blobs = []
    for b in blobs:
        buf = np.full(b.size + 512, 0xA5, dtype=np.uint8)
        buf[256:256 + b.size] = b
        dev_blobs.append(to_dev(buf))
    table = torch.tensor([t.data_ptr() + 256 for t in dev_blobs], dtype=torch.int64, device="cuda")
    x, w = to_dev(x16), to_dev(w16)
    acts = dev_zeros_u16(K * F + 16, fill=0x7BFF)
    y = dev_zeros_u16(D + 16, fill=0x7BFF)
    res = dev_zeros_u16(D)
    moe = MoE(tf_ctx)
    coff = capi_offsets(off)
    moe.encode_routed_phase1(table, coff, x, acts, D, F, K)
    moe.encode_routed_phase2_reduce(table, coff, acts, w, res, y, D, F, K)
    torch.cuda.synchronize()
    acts_h, y_h = from_dev(acts, np.uint16), from_dev(y, np.uint16)
    assert np.all(acts_h[K * F:] == 0x7BFF) and np.all(y_h[D:] == 0x7BFF)
    y_truth16, y_truth, acts_truth = o.moe_routed_decode(blobs, off, x16, w16, from_dev(res, np.uint16), D, F, order=0)
    assert o.rel_error(o.f16_to_f32(acts_h[:K * F]), o.f16_to_f32(acts_truth.reshape(-1))) < FP16_CHAINED
    assert o.rel_error(o.f16_to_f32(y_h[:D]), y_truth) < FP16_CHAINED
    assert o.rel_l2(o.f16_to_f32(y_h[:D]), y_truth) < FP16_CHAINED

    # hit/miss split == full, bitwise (MoEFusedFFNTests.swift:154-156)
    acts2 = dev_zeros_u16(K * F)
    hits = to_dev(np.array([0, 3, 5], dtype=np.uint32))
    misses = to_dev(np.array([1, 2, 4, 6, 7], dtype=np.uint32))
    moe.encode_routed_phase1_subset(table, coff, x, acts2, D, F, K, hits, 3)
    moe.encode_routed_phase1_subset(table, coff, x, acts2, D, F, K, misses, 5)
    torch.cuda.synchronize()
    assert from_dev(acts2, np.uint16).tobytes() == acts_h[:K * F].tobytes()

    # a non-zero residual is added in fp32 before the single rounding (moe.metal:475-480)
    res2 = to_dev(o.f32_to_f16(np.linspace(-1, 1, D).astype(np.float32)))
    moe.encode_routed_phase2_reduce(table, coff, acts, w, res2, y, D, F, K)
    torch.cuda.synchronize()
    _, y_truth2, _ = o.moe_routed_decode(blobs, off, x16, w16, from_dev(res2, np.uint16), D, F, order=0)
    assert o.rel_error(o.f16_to_f32(from_dev(y, np.uint16)[:D]), y_truth2) < FP16_CHAINED


def test_routed_decode_production_shape_with_device_table(tf_ctx, oracle):
    """benchmark configuration 1 routed half: D=2816, F=704, 8 of 16 pooled experts chosen by ids on the device."""
    import torch
    from turbo_fieldfare_b200.kernels import MoE
    o = oracle
    D, F, K, E = 2816, 704, 8, 16
    rng = np.random.default_rng(77)
    off, payload, stride = o.blob_layout(D, F)
    assert stride == 3358720
    pool_h = np.zeros(E * stride, dtype=np.uint8)
    for e in range(E):
        pool_h[e * stride:(e + 1) * stride] = random_blob(o, D, F, rng, off, stride)[0]
    pool = to_dev(pool_h)
    ids = np.array([9, 2, 15, 0, 7, 11, 4, 200], dtype=np.uint32)       # 200 clamps to E-1
    x16 = o.f32_to_f16(rng.standard_normal(D).astype(np.float32))
    w16 = o.f32_to_f16(rng.dirichlet(np.ones(K)).astype(np.float32))
    table = torch.zeros(K, dtype=torch.int64, device="cuda")
    moe = MoE(tf_ctx)
    moe.encode_expert_table(pool, stride, to_dev(ids), K, E, table)
    acts, y = dev_zeros_u16(K * F), dev_zeros_u16(D)
    coff = capi_offsets(off)
    moe.encode_routed_phase1(table, coff, to_dev(x16), acts, D, F, K)
    moe.encode_routed_phase2_reduce(table, coff, acts, to_dev(w16), None, y, D, F, K)
    torch.cuda.synchronize()
    clamped = np.minimum(ids, E - 1)
    assert table.cpu().tolist() == [pool.data_ptr() + int(e) * stride for e in clamped]
    blobs = [pool_h[int(e) * stride:(int(e) + 1) * stride] for e in clamped]
    _, y_truth, acts_truth = o.moe_routed_decode(blobs, off, x16, w16, None, D, F, order=0)
    assert o.rel_l2(o.f16_to_f32(from_dev(acts, np.uint16)), o.f16_to_f32(acts_truth.reshape(-1))) < FP16_CHAINED
    assert o.rel_l2(o.f16_to_f32(from_dev(y, np.uint16)), y_truth) < FP16_CHAINED
    assert o.rel_error(o.f16_to_f32(from_dev(y, np.uint16)), y_truth) < FP16_CHAINED


# ---------------------------------------------------------------------------
# shared expert, norms
# ---------------------------------------------------------------------------

def _shared_run(tf_ctx, o, gate, up, down, x16):
    import torch
    from turbo_fieldfare_b200.kernels import SharedExpertInt4, SharedExpertProjection
    D, Fs = gate.n, gate.m
    proj = lambda m: SharedExpertProjection(to_dev(m.packed), to_dev(m.scales), to_dev(m.biases), m.m, m.n)
    y = dev_zeros_u16(D)
    sg, su, sa = dev_zeros_u16(Fs), dev_zeros_u16(Fs), dev_zeros_u16(Fs)
    SharedExpertInt4(tf_ctx).encode(to_dev(x16), proj(gate), proj(up), proj(down), y, sg, su, sa)
    torch.cuda.synchronize()
    return from_dev(y, np.uint16)


def test_shared_expert_reference_fixture(tf_ctx, oracle):
    # Tests/TurboFieldfare/Core/Kernels/MoE/SharedExpertInt4Tests.swift:11-52 (D=128, F=64, seed 0x604; rel < 6e-3)
    o = oracle
    D, Fs = 128, 64
    rng = o.SplitMix64(0x604)
    gate = o.quantize_rows(np.stack([rng.uniform_array(-0.5, 0.5, D) for _ in range(Fs)]), 4)
    up = o.quantize_rows(np.stack([rng.uniform_array(-0.5, 0.5, D) for _ in range(Fs)]), 4)
    down = o.quantize_rows(np.stack([rng.uniform_array(-0.5, 0.5, Fs) for _ in range(D)]), 4)
    x16 = o.f32_to_f16(rng.uniform_array(-1.0, 1.0, D))
    y = _shared_run(tf_ctx, o, gate, up, down, x16)
    _, truth = o.shared_expert_int4(gate, up, down, x16, order=0)
    assert o.rel_error(o.f16_to_f32(y), truth) < 6e-3


def test_shared_expert_production_shape(tf_ctx, oracle):
    o = oracle
    rng = np.random.default_rng(99)
    D, Fs = 2816, 2112
    gate, up, down = config0_matrix(o, Fs, D, rng), config0_matrix(o, Fs, D, rng), config0_matrix(o, D, Fs, rng)
    x16 = o.f32_to_f16(rng.standard_normal(D).astype(np.float32))
    y = _shared_run(tf_ctx, o, gate, up, down, x16)
    _, truth = o.shared_expert_int4(gate, up, down, x16, order=0)
    assert o.rel_l2(o.f16_to_f32(y), truth) < FP16_CHAINED


def _shared_int8_reference(o, gate, up, down, x16):
    """SharedExpertInt8Tests.swift:62-75: gate and up by the GEMV reference, act = half(gelu(g) * u), then down.
    (The kernel also rounds gate and up to fp16 before the activation, dequant_int8.metal:148-152; both forms sit well
    inside the bound.)"""
    x = o.f16_to_f32(x16)
    g, u = o.gemv_ref(gate, x), o.gemv_ref(up, x)
    inner = 0.7978845608028654 * (g.astype(np.float64) + 0.044715 * g.astype(np.float64) ** 3)
    act = o.f32_to_f16((0.5 * g.astype(np.float64) * (1.0 + np.tanh(inner))).astype(np.float32) * u)
    return o.gemv_ref(down, o.f16_to_f32(act))


def _shared_int8_run(tf_ctx, o, gate, up, down, x16_rows, w_off=0):
    import ctypes as C
    import torch
    from turbo_fieldfare_b200.kernels import SharedExpertProjection, _ptr
    T, D = x16_rows.shape
    Fs = gate.m

    def proj(m):
        w = np.zeros(w_off + m.packed.size, dtype=np.uint8)
        w[w_off:] = m.packed.reshape(-1)
        return SharedExpertProjection(to_dev(w), to_dev(m.scales), to_dev(m.biases), m.m, m.n, weights_offset=w_off)

    pg, pu, pd = proj(gate), proj(up), proj(down)
    y = dev_zeros_u16(T * D, fill=0x7E00)
    scratch = dev_zeros_u16(T * Fs)
    g, u, dn = pg.c_struct(), pu.c_struct(), pd.c_struct()
    tf_ctx.check(tf_ctx.lib.tf_shared_expert_int8_block(tf_ctx.handle, 0, _ptr(to_dev(x16_rows)), 0, D, C.byref(g), C.byref(u), C.byref(dn),
                                                        _ptr(y), 0, D, _ptr(scratch), T))
    torch.cuda.synchronize()
    return from_dev(y, np.uint16).reshape(T, D)


def test_shared_expert_int8_reference_fixture(tf_ctx, oracle):
    # Tests/TurboFieldfare/Core/Kernels/MoE/SharedExpertInt8Tests.swift:49-118 (D=128, F=64, seed 0x601; rel < 4e-3)
    o = oracle
    D, Fs = 128, 64
    rng = o.SeedTree(0x601).key("shared-expert-int8")
    x16 = o.f32_to_f16(rng.uniform_array(-0.4, 0.4, D))
    gate = o.quantize_rows(np.stack([rng.uniform_array(-0.4, 0.4, D) for _ in range(Fs)]), 8)
    up = o.quantize_rows(np.stack([rng.uniform_array(-0.4, 0.4, D) for _ in range(Fs)]), 8)
    down = o.quantize_rows(np.stack([rng.uniform_array(-0.4, 0.4, Fs) for _ in range(D)]), 8)
    y = _shared_int8_run(tf_ctx, o, gate, up, down, x16[None, :])
    assert o.rel_error(o.f16_to_f32(y[0]), _shared_int8_reference(o, gate, up, down, x16)) < 4e-3


@pytest.mark.parametrize("T,w_off", [(1, 0), (5, 0), (70, 3)])
def test_shared_expert_int8_block_production_shape(tf_ctx, oracle, T, w_off):
    """The 8-bit shared expert at production width for a block of rows (PrefillSharedExpert loops the rows,
    Kernels/Prefill/MoE/PrefillSharedExpert.swift:11-59), packed planes at an odd byte offset included."""
    o = oracle
    rng = np.random.default_rng(500 + T)
    D, Fs = 2816, 2112
    gate, up, down = (config0_matrix(o, Fs, D, rng, bits=8), config0_matrix(o, Fs, D, rng, bits=8), config0_matrix(o, D, Fs, rng, bits=8))
    x16 = o.f32_to_f16(rng.standard_normal((T, D)).astype(np.float32))
    y = _shared_int8_run(tf_ctx, o, gate, up, down, x16, w_off)
    assert np.isfinite(o.f16_to_f32(y)).all()
    for t in sorted({0, T // 2, T - 1}):
        assert o.rel_l2(o.f16_to_f32(y[t]), _shared_int8_reference(o, gate, up, down, x16[t])) < FP16_CHAINED


def test_shared_expert_int8_errors(tf_ctx):
    import ctypes as C
    import torch
    from turbo_fieldfare_b200.kernels import SharedExpertProjection, _ptr
    b = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = lambda r, c: SharedExpertProjection(b, b, b, r, c).c_struct()
    g, u, d_bad, d_ok = p(64, 128), p(64, 128), p(128, 128), p(128, 64)
    call = lambda dn: tf_ctx.lib.tf_shared_expert_int8_block(tf_ctx.handle, 0, _ptr(b), 0, 128, C.byref(g), C.byref(u), C.byref(dn),
                                                             _ptr(b), 0, 128, _ptr(b), 1)
    assert call(d_bad) == 7                      # SharedExpertInt8Error.dimensionMismatch (SharedExpertInt8.swift:84-88)
    assert call(d_ok) == 0
    torch.cuda.synchronize()


def test_shared_expert_errors(tf_ctx, oracle):
    import torch
    from turbo_fieldfare_b200.kernels import SharedExpertInt4, SharedExpertProjection, TFError
    b = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    small = torch.zeros(8, dtype=torch.uint8, device="cuda")
    p = lambda r, c: SharedExpertProjection(b, b, b, r, c)
    k = SharedExpertInt4(tf_ctx)
    with pytest.raises(TFError) as e:          # SharedExpertError.dimensionMismatch
        k.encode(b, p(64, 128), p(64, 128), p(128, 128), b, b, b, b)
    assert e.value.status == 7
    with pytest.raises(TFError) as e:          # SharedExpertError.scratchTooSmall
        k.encode(b, p(64, 128), p(64, 128), p(128, 64), b, small, b, b)
    assert e.value.status == 6


def test_rmsnorm_and_layer_tail(tf_ctx, oracle):
    import torch
    from turbo_fieldfare_b200.kernels import FusedLayerTail, RMSNorm
    o = oracle
    rng = np.random.default_rng(3)
    T, D, stride = 5, 2816, 2816 + 8
    x = np.zeros((T, stride), dtype=np.float32)
    x[:, :D] = rng.standard_normal((T, D))
    x16 = o.f32_to_f16(x)
    w = o.f32_to_bf16((1 + 0.02 * rng.standard_normal(D)).astype(np.float32))
    y = dev_zeros_u16(T * stride)
    RMSNorm(tf_ctx).encode(to_dev(x16), to_dev(w), y, T, D, stride)
    y0 = dev_zeros_u16(T * stride)
    RMSNorm(tf_ctx).encode(to_dev(x16), None, y0, T, D, stride)
    torch.cuda.synchronize()
    got = o.f16_to_f32(from_dev(y, np.uint16).reshape(T, stride)[:, :D])
    ref = o.f16_to_f32(o.rmsnorm(np.ascontiguousarray(x16[:, :D]), w))
    assert o.rel_error(got, ref) < 2e-3
    assert np.all(from_dev(y, np.uint16).reshape(T, stride)[:, D:] == 0)     # padding untouched
    got0 = o.f16_to_f32(from_dev(y0, np.uint16).reshape(T, stride)[:, :D])
    assert o.rel_error(got0, o.f16_to_f32(o.rmsnorm(np.ascontiguousarray(x16[:, :D]), None))) < 2e-3

    h2 = o.f32_to_f16(rng.standard_normal((T, D)).astype(np.float32))
    h1 = o.f32_to_f16(rng.standard_normal((T, D)).astype(np.float32))
    hid = o.f32_to_f16(rng.standard_normal((T, D)).astype(np.float32))
    w2 = o.f32_to_bf16((1 + 0.02 * rng.standard_normal(D)).astype(np.float32))
    hd = to_dev(hid)
    FusedLayerTail(tf_ctx).encode(to_dev(h2), to_dev(h1), hd, to_dev(w2), to_dev(w), T, D, D, 1e-6, 0.75)
    torch.cuda.synchronize()
    ref = o.f16_to_f32(o.layer_tail(h2, h1, hid, w2, w, 1e-6, 0.75))
    assert o.rel_error(o.f16_to_f32(from_dev(hd, np.uint16).reshape(T, D)), ref) < 3e-3


def _lm_head_gpu(tf_ctx, o, hidden16, norm, mat, d, v, hidden_offset=0):
    import torch
    from turbo_fieldfare_b200.kernels import LMHeadChainInt4
    out = torch.full((1,), 0xFFFF, dtype=torch.int32, device="cuda")
    LMHeadChainInt4(tf_ctx).encode_greedy_decode(to_dev(hidden16), to_dev(norm), to_dev(mat.packed), to_dev(mat.scales),
                                                 to_dev(mat.biases), out, d, v, hidden_offset=hidden_offset)
    torch.cuda.synchronize()
    return int(out.cpu().numpy().view(np.uint32)[0])


def _constant_rows(o, values, d):
    return o.quantize_rows(np.repeat(np.asarray(values, dtype=np.float32)[:, None], d, axis=1), 4)


def test_lm_head_greedy_reference_cases(tf_ctx, oracle):
    """The five cases of Tests/TurboFieldfare/Core/Kernels/Fusions/LMHeadChainInt4Tests.swift:113-224."""
    o = oracle
    d, v = 64, 1024
    # raw greedy == CPU reference, seed 0x1A4E4EAD20260603
    rng = o.SplitMix64(0x1A4E4EAD20260603)
    hidden = o.f32_to_f16(rng.uniform_array(-1, 1, d))
    norm = o.f32_to_bf16(rng.uniform_array(0.5, 1.5, d))
    mat = o.quantize_rows(np.stack([rng.uniform_array(-1, 1, d) for _ in range(v)]), 4)
    want, _ = o.lm_head_greedy(hidden, norm, mat)
    assert _lm_head_gpu(tf_ctx, o, hidden, norm, mat, d, v) == want
    ones = o.f32_to_bf16(np.ones(d, np.float32))
    # every candidate invalid -> token 0
    nan_hidden = np.full(d, 0x7E00, dtype=np.uint16)
    assert _lm_head_gpu(tf_ctx, o, nan_hidden, ones, _constant_rows(o, [0.25] * v, d), d, v) == 0
    # vocabulary sizes
    for vv in (1024, 2048, 4096):
        target = vv - 3
        hid = o.f32_to_f16(np.array([0.25 + (i % 7) * 0.01 for i in range(d)], np.float32))
        rows = _constant_rows(o, [1.0 if r == target else -0.5 for r in range(vv)], d)
        want, _ = o.lm_head_greedy(hid, ones, rows)
        assert want == target
        assert _lm_head_gpu(tf_ctx, o, hid, ones, rows, d, vv) == want
    # ties resolve to the lowest index
    hid = o.f32_to_f16(np.array([0.2 + (i % 5) * 0.02 for i in range(d)], np.float32))
    rows = _constant_rows(o, [1.0 if r in (17, 311) else -0.25 for r in range(v)], d)
    assert _lm_head_gpu(tf_ctx, o, hid, ones, rows, d, v) == 17
    # the hidden offset selects a row of a strided buffer
    stride, selected, target = d + 16, 3, 777
    buf = np.zeros((5, stride), dtype=np.float32)
    for r in range(5):
        buf[r, :d] = [0.25 + (i % 7) * 0.01 if r == selected else -0.4 - (i % 5) * 0.01 for i in range(d)]
    rows = _constant_rows(o, [1.0 if r == target else -0.25 for r in range(v)], d)
    assert _lm_head_gpu(tf_ctx, o, o.f32_to_f16(buf), ones, rows, d, v, hidden_offset=selected * stride * 2) == target


def test_lm_head_greedy_streaming_shape(tf_ctx, oracle):
    """A vocabulary large enough for the tensor-core streaming GEMV (>= 4096 rows, D = 2816), ragged last block; the
    context's scratch grows between calls. The chosen row must hold the oracle's maximum up to fp32 summation order."""
    o = oracle
    d = 2816
    rng = np.random.default_rng(77)
    for v in (5000, 16384 + 40):
        mat = config0_matrix(o, v, d, rng)
        hidden = o.f32_to_f16(rng.standard_normal(d).astype(np.float32))
        norm = o.f32_to_bf16((1 + 0.1 * rng.standard_normal(d)).astype(np.float32))
        want, logits = o.lm_head_greedy(hidden, norm, mat)
        got = _lm_head_gpu(tf_ctx, o, hidden, norm, mat, d, v)
        assert got == want or abs(float(logits[got]) - float(logits[want])) <= 1e-5 * max(1.0, abs(float(logits[want]))), (got, want)
    assert tf_ctx.device_status() == 0


def test_post_attention_setup_equals_the_primitive_chain_bitwise(tf_ctx, oracle):
    """The reference's own test of this fusion (FusedPostAttentionSetupTests.swift:11-108): seed 0x9057A77E, D = 2816,
    uniform inputs; the fused kernel equals rmsnorm -> add -> rmsnorm x 3 bit for bit. The CPU chain of the oracle
    (another summation order) bounds it as well."""
    import torch
    from turbo_fieldfare_b200.kernels import FusedPostAttentionSetup, RMSNorm
    o = oracle
    D = 2816
    rng = o.SplitMix64(0x9057A77E)
    hidden = o.f32_to_f16(rng.uniform_array(-1.0, 1.0, D))
    attn = o.f32_to_f16(rng.uniform_array(-1.0, 1.0, D))
    w_post, w_pre, w_pre2 = (o.f32_to_bf16(rng.uniform_array(0.5, 1.5, D)) for _ in range(3))
    dw_post, dw_pre, dw_pre2 = to_dev(w_post), to_dev(w_pre), to_dev(w_pre2)
    rms = RMSNorm(tf_ctx)
    # primitive chain on the device; the fp16 add on the host, as in the reference's test
    attn_legacy = to_dev(attn.copy())
    rms.encode(attn_legacy, dw_post, attn_legacy, 1, D)
    torch.cuda.synchronize()
    hidden_legacy = o.f32_to_f16((o.f16_to_f32(hidden) + o.f16_to_f32(from_dev(attn_legacy, np.uint16))).astype(np.float32))
    hl = to_dev(hidden_legacy)
    dense_l, routed_l, router_l = dev_zeros_u16(D), dev_zeros_u16(D), dev_zeros_u16(D)
    rms.encode(hl, dw_pre, dense_l, 1, D)
    rms.encode(hl, dw_pre2, routed_l, 1, D)
    rms.encode(hl, None, router_l, 1, D)
    hf, af = to_dev(hidden.copy()), to_dev(attn.copy())
    dense_f, routed_f, router_f = dev_zeros_u16(D), dev_zeros_u16(D), dev_zeros_u16(D)
    FusedPostAttentionSetup(tf_ctx).encode(hf, af, dense_f, routed_f, router_f, dw_post, dw_pre, dw_pre2, D, 1e-6)
    torch.cuda.synchronize()
    assert np.array_equal(from_dev(hf, np.uint16), hidden_legacy)
    assert np.array_equal(from_dev(dense_f, np.uint16), from_dev(dense_l, np.uint16))
    assert np.array_equal(from_dev(routed_f, np.uint16), from_dev(routed_l, np.uint16))
    assert np.array_equal(from_dev(router_f, np.uint16), from_dev(router_l, np.uint16))
    assert np.array_equal(from_dev(af, np.uint16), attn)                        # attn is an input only
    ref = o.post_attn_setup(hidden, attn, w_post, w_pre, w_pre2)
    for got, want in zip((hf, dense_f, routed_f, router_f), ref):
        assert o.rel_error(o.f16_to_f32(from_dev(got, np.uint16)), o.f16_to_f32(want.reshape(-1))) < 2e-3


def test_post_attention_setup_block_form_with_row_strides(tf_ctx, oracle):
    """The prefill form: T rows, a separate stride per buffer (Metal/Prefill/prefill.metal:178-254); padding untouched."""
    import torch
    from turbo_fieldfare_b200.kernels import FusedPostAttentionSetup
    o = oracle
    rng = np.random.default_rng(41)
    T, D = 7, 2816
    strides = dict(hidden=D + 8, attn=D + 24, dense=D, routed=D + 16, router=D + 40)
    def rows(stride, fill):
        a = np.full((T, stride), fill, dtype=np.uint16)
        a[:, :D] = o.f32_to_f16(rng.standard_normal((T, D)).astype(np.float32))
        return a
    hidden, attn = rows(strides["hidden"], 0x1234), rows(strides["attn"], 0x4321)
    w = [o.f32_to_bf16((1 + 0.1 * rng.standard_normal(D)).astype(np.float32)) for _ in range(3)]
    hd, ad = to_dev(hidden.copy()), to_dev(attn.copy())
    outs = {k: to_dev(np.full((T, strides[k]), 0x7777, dtype=np.uint16)) for k in ("dense", "routed", "router")}
    FusedPostAttentionSetup(tf_ctx).encode(hd, ad, outs["dense"], outs["routed"], outs["router"], to_dev(w[0]), to_dev(w[1]),
                                           to_dev(w[2]), D, 1e-6, rows=T, hidden_stride=strides["hidden"],
                                           attn_stride=strides["attn"], dense_stride=strides["dense"],
                                           routed_stride=strides["routed"], router_stride=strides["router"])
    torch.cuda.synchronize()
    ref = o.post_attn_setup(np.ascontiguousarray(hidden[:, :D]), np.ascontiguousarray(attn[:, :D]), *w)
    got_hidden = from_dev(hd, np.uint16).reshape(T, strides["hidden"])
    assert o.rel_error(o.f16_to_f32(got_hidden[:, :D]), o.f16_to_f32(ref[0])) < 2e-3
    assert np.all(got_hidden[:, D:] == 0x1234)
    for k, want in zip(("dense", "routed", "router"), ref[1:]):
        got = from_dev(outs[k], np.uint16).reshape(T, strides[k])
        assert o.rel_error(o.f16_to_f32(got[:, :D]), o.f16_to_f32(want)) < 2e-3, k
        assert np.all(got[:, D:] == 0x7777), k


@pytest.mark.parametrize("m,n,sb", [(4096, 256, 0), (4224, 2816, 0), (5000, 2816, 1)])
def test_int4_gemv_streaming_kernel_for_large_matrices(tf_ctx, oracle, m, n, sb):
    """Matrices of at least 4096 rows with 16-byte aligned planes take the tensor-core streaming kernel; same bound as
    the reference's GEMV tests (rel < 5e-3, Tests/TurboFieldfare/Core/Kernels/Quant/DequantInt4GEMVTests.swift:41-128),
    ragged last block of rows included, both scale dtypes."""
    import torch
    from turbo_fieldfare_b200.kernels import DequantInt4GEMV
    o = oracle
    rng = np.random.default_rng(m + n + sb)
    mat = config0_matrix(o, m, n, rng, sb_dtype=sb)
    x16 = o.f32_to_f16(rng.standard_normal(n).astype(np.float32))
    y = dev_zeros_u16(m, fill=0x7E00)
    DequantInt4GEMV(tf_ctx).encode(to_dev(mat.packed), to_dev(mat.scales), to_dev(mat.biases), to_dev(x16), y, m, n,
                                   sb_dtype=sb)
    torch.cuda.synchronize()
    got = o.f16_to_f32(from_dev(y, np.uint16))
    ref = o.gemv_ref(mat, o.f16_to_f32(x16))
    assert np.isfinite(got).all()
    assert o.rel_error(got, ref) < 5e-3


@pytest.mark.parametrize("m,n,count,shared_x", [(704, 2816, 7, True), (704, 2816, 3, False), (72, 256, 5, True), (96, 192, 4, False)])
def test_int4_gemv_batched_over_expert_blobs(tf_ctx, oracle, m, n, count, shared_x):
    """One launch over the same tensor of consecutive expert blobs (config-0 matrices 704 x 2816 at the blob stride)
    equals one tf_int4_gemv per matrix bit for bit where both run the same kernel family, and the oracle within the
    GEMV tolerance; n = 192 takes the per-matrix fallback."""
    import torch
    from turbo_fieldfare_b200.kernels import DequantInt4GEMV
    o = oracle
    rng = np.random.default_rng(m + n + count)
    mats = [config0_matrix(o, m, n, rng) for _ in range(count)]
    w_bytes, sb_bytes = m * n // 2, m * (n // 64) * 2
    s_off = (w_bytes + 255) // 256 * 256
    b_off = s_off + (sb_bytes + 255) // 256 * 256
    stride = (b_off + sb_bytes + 16383) // 16384 * 16384
    blob = np.zeros(count * stride, dtype=np.uint8)
    for b, mat in enumerate(mats):
        blob[b * stride:b * stride + w_bytes] = mat.packed.reshape(-1)
        blob[b * stride + s_off:b * stride + s_off + sb_bytes] = mat.scales.view(np.uint8).reshape(-1)
        blob[b * stride + b_off:b * stride + b_off + sb_bytes] = mat.biases.view(np.uint8).reshape(-1)
    xs = o.f32_to_f16(rng.standard_normal((1 if shared_x else count, n)).astype(np.float32))
    dev = to_dev(blob)
    x = to_dev(xs)
    y = dev_zeros_u16(count * m, fill=0x7E00)
    op = DequantInt4GEMV(tf_ctx)
    before = tf_ctx.launch_count
    op.encode_batched(dev, dev, dev, stride, x, y, m, n, count, scales_offset=s_off, biases_offset=b_off,
                      x_stride_elements=0 if shared_x else n)
    torch.cuda.synchronize()
    assert tf_ctx.launch_count - before == (1 if n % 256 == 0 else count)
    got = from_dev(y, np.uint16).reshape(count, m)
    for b, mat in enumerate(mats):
        xb = xs[0 if shared_x else b]
        ref = o.gemv_ref(mat, o.f16_to_f32(xb))
        assert o.rel_error(o.f16_to_f32(got[b]), ref) < FP16_REDUCTION, b
        y1 = dev_zeros_u16(m)
        op.encode(dev, dev, dev, to_dev(xb), y1, m, n, weights_offset=b * stride, scales_offset=b * stride + s_off,
                  biases_offset=b * stride + b_off)
        torch.cuda.synchronize()
        assert o.rel_error(o.f16_to_f32(got[b]), o.f16_to_f32(from_dev(y1, np.uint16))) < 2e-3, b
