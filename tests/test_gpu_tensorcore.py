"""GPU parity of the tcgen05 / TMEM kernels: the dense int4 QMM, the grouped routed experts over
expert-sorted rows and the shared expert block, each against the CPU oracle and against the
CUDA-core kernels of the same operators."""
import numpy as np
import pytest

from helpers import capi_offsets, config0_matrix, dev_zeros_u16, from_dev, random_blob, to_dev

pytestmark = pytest.mark.gpu
QMM_TOL = 1e-3          # MPPPrefillInt4QMMTests.swift:180-185: relative <= 1e-3 against the CPU reference
FP16_CHAINED = 1e-2


def _status_ok(tf_ctx):
    assert tf_ctx.device_status() == 0, "a kernel abandoned a bounded wait"


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (32, 128, 128), (128, 128, 256), (200, 136, 192), (129, 704, 2816),
                                   (512, 2816, 704)])
def test_int4_qmm_vs_oracle(tf_ctx, oracle, M, N, K):
    import torch
    from turbo_fieldfare_b200.kernels import MPPPrefillInt4QMM
    o = oracle
    rng = np.random.default_rng(M * 31 + N * 7 + K)
    mat = config0_matrix(o, N, K, rng)
    x16 = o.f32_to_f16(rng.standard_normal((M, K)).astype(np.float32))
    y = dev_zeros_u16(M * N, fill=0x7E00)
    MPPPrefillInt4QMM(tf_ctx).encode(to_dev(mat.packed), to_dev(mat.scales), to_dev(mat.biases), to_dev(x16), y, M, N, K)
    torch.cuda.synchronize()
    _status_ok(tf_ctx)
    got = o.f16_to_f32(from_dev(y, np.uint16).reshape(M, N))
    ref = o.int4_qmm_ref(mat, x16)
    assert np.isfinite(got).all()
    assert o.rel_l2(got, ref) < QMM_TOL
    assert o.rel_error(got, ref) < QMM_TOL


def test_int4_qmm_reports_fallback_like_the_reference(tf_ctx):
    """MPPPrefillInt4QMMTests.swift:287-318: an unsupported K and an odd scale offset report `.unavailable`
    (nothing is launched); the call without a path argument returns an error status for the same inputs."""
    from turbo_fieldfare_b200.kernels import MPPPrefillInt4QMM, TFError
    z = dev_zeros_u16(4096)
    op = MPPPrefillInt4QMM(tf_ctx)
    before = tf_ctx.launch_count
    assert op.encode(z, z, z, z, z, 1, 1, 65) == "unavailable"
    assert op.encode(z, z, z, z, z, 1, 1, 64, weights_offset=1, scales_offset=1) == "unavailable"
    assert tf_ctx.launch_count == before
    from turbo_fieldfare_b200.kernels import _ptr
    with pytest.raises(TFError):
        tf_ctx.check(tf_ctx.lib.tf_int4_qmm(tf_ctx.handle, 0, _ptr(z), 0, _ptr(z), 0, _ptr(z), 0, _ptr(z), 0, _ptr(z), 0, 4, 64, 96))


def _mpp_inputs(o, m, n, k, adversarial):
    """The closed-form inputs of MPPPrefillInt4QMMTests.swift:20-63: packed byte = index * 37 + 0x29, scale and bias
    cycles (the adversarial table holds a negative scale and the bf16 denormals 0x0001 / 0x8001), x = ((11 i) % 29 - 14) / 64."""
    groups = k // 64
    packed = ((np.arange(n * k // 2, dtype=np.uint64) * 37 + 0x29) & 0xFF).astype(np.uint8).reshape(n, k // 2)
    row, grp = np.meshgrid(np.arange(n), np.arange(groups), indexing="ij")
    f32 = np.float32
    if adversarial:
        st = np.array([o.f32_to_bf16(np.array([0.001], f32))[0], o.f32_to_bf16(np.array([-0.0015], f32))[0], 0x0001, 0x8001], dtype=np.uint16)
        bt = np.array([o.f32_to_bf16(np.array([-0.01], f32))[0], o.f32_to_bf16(np.array([0.006], f32))[0], 0x0001, 0x8001], dtype=np.uint16)
        scales, biases = st[(row + grp) % 4], bt[(row * 3 + grp) % 4]
    else:
        scales = o.f32_to_bf16((f32(0.001) + ((row + grp) % 5).astype(f32) * f32(0.00025)).astype(f32))
        biases = o.f32_to_bf16((f32(-0.01) + ((row * 3 + grp) % 7).astype(f32) * f32(0.002)).astype(f32))
    idx = np.arange(m * k, dtype=np.int64)
    x16 = o.f32_to_f16((((idx * 11) % 29 - 14).astype(f32) / f32(64.0)).reshape(m, k))
    return np.ascontiguousarray(packed), np.ascontiguousarray(scales.astype(np.uint16)), np.ascontiguousarray(biases.astype(np.uint16)), x16


def _mpp_cpu_reference(o, packed, scales, biases, x16, m, n, k):
    """cpuReference of MPPPrefillInt4QMMTests.swift:80-105: weight = float(q) * scale + bias in fp32, fused
    multiply-add accumulation over k in fp32, result rounded to fp16."""
    codes = np.empty((n, k), dtype=np.float32)
    codes[:, 0::2] = packed & 0x0F
    codes[:, 1::2] = packed >> 4
    s = np.repeat(o.bf16_to_f32(scales), 64, axis=1)
    b = np.repeat(o.bf16_to_f32(biases), 64, axis=1)
    with np.errstate(under="ignore"):
        w = ((codes * s).astype(np.float32) + b).astype(np.float32)
    x = o.f16_to_f32(x16)
    acc = np.zeros((m, n), dtype=np.float32)
    for c in range(k):     # one fma per step: the product is exact in double, one rounding back to fp32
        acc = (np.outer(x[:, c].astype(np.float64), w[:, c].astype(np.float64)) + acc.astype(np.float64)).astype(np.float32)
    return o.f16_to_f32(o.f32_to_f16(acc))


@pytest.mark.parametrize("m,n,k,adversarial,offsets,path", [
    (64, 32, 64, False, (0, 0, 0), "affine-threadgroup-f16"),
    (64, 32, 128, True, (0, 0, 0), "affine-threadgroup-f16"),
    (17, 35, 64, False, (0, 0, 0), "cuda-cores"),
    (17, 35, 128, True, (13, 2, 6), "cuda-cores"),
    (32, 1024, 2816, False, (0, 0, 0), "affine-threadgroup-f16"),      # "full-kv", a production attention shape (:208-215)
    (128, 64, 256, True, (0, 0, 0), "affine-threadgroup-f16"),
])
def test_int4_qmm_reference_closed_form_fixture(tf_ctx, oracle, m, n, k, adversarial, offsets, path):
    """The reference's own QMM fixture and bounds (MPPPrefillInt4QMMTests.swift:173-186): max-abs <= 0.03 and
    relative <= 1e-3 against its CPU reference, including the shape with odd N and the (13, 2, 6)-byte plane offsets."""
    import torch
    from turbo_fieldfare_b200.kernels import MPPPrefillInt4QMM
    o = oracle
    packed, scales, biases, x16 = _mpp_inputs(o, m, n, k, adversarial)
    w_off, s_off, b_off = offsets

    def with_prefix(a, prefix):
        raw = np.zeros(prefix + a.nbytes, dtype=np.uint8)
        raw[prefix:] = a.view(np.uint8).reshape(-1)
        return to_dev(raw)

    y = dev_zeros_u16(m * n, fill=0x7E00)
    got_path = MPPPrefillInt4QMM(tf_ctx).encode(with_prefix(packed, w_off), with_prefix(scales, s_off), with_prefix(biases, b_off),
                                                to_dev(x16), y, m, n, k, weights_offset=w_off, scales_offset=s_off,
                                                biases_offset=b_off)
    torch.cuda.synchronize()
    _status_ok(tf_ctx)
    assert got_path == path
    got = o.f16_to_f32(from_dev(y, np.uint16).reshape(m, n))
    ref = _mpp_cpu_reference(o, packed, scales, biases, x16, m, n, k)
    assert np.isfinite(got).all()
    assert float(np.max(np.abs(got - ref))) <= 0.03
    assert o.rel_error(got, ref) <= 1e-3
    # and against the oracle's double-accumulated form of the same reference
    mat = o.AffineMatrix(packed, scales, biases, 4, k)
    assert o.rel_error(got, o.int4_qmm_ref(mat, x16)) <= 1e-3


def test_int4_qmm_is_byte_stable_across_dispatches(tf_ctx, oracle):
    """MPPPrefillInt4QMMTests.swift:236-285: the production shape M=32, N=2816, K=8192 gives identical bytes on
    every one of 32 dispatches."""
    import torch
    from turbo_fieldfare_b200.kernels import MPPPrefillInt4QMM
    o = oracle
    m, n, k = 32, 2816, 8192
    packed, scales, biases, x16 = _mpp_inputs(o, m, n, k, False)
    W, S, B, X = to_dev(packed), to_dev(scales), to_dev(biases), to_dev(x16)
    outs = dev_zeros_u16(32 * m * n, fill=0x7E00)
    op = MPPPrefillInt4QMM(tf_ctx)
    for run in range(32):
        assert op.encode(W, S, B, X, outs, m, n, k, y_offset=run * m * n * 2) == "affine-threadgroup-f16"
    torch.cuda.synchronize()
    _status_ok(tf_ctx)
    got = from_dev(outs, np.uint16).reshape(32, m * n)
    assert (got == got[0]).all()
    mat = o.AffineMatrix(packed, scales, biases, 4, k)
    assert o.rel_error(o.f16_to_f32(got[0]).reshape(m, n), o.int4_qmm_ref(mat, x16)) <= 1e-3


@pytest.mark.parametrize("M,N,K", [(96, 128, 256), (300, 704, 2816)])
def test_int4_qmm_quantiser_built_planes(tf_ctx, oracle, M, N, K):
    """Weights U(-0.5, 0.5) through the reference's quantiser (scale about 1/15, above 2^-5): the wide-scale branch of
    the dequantiser, which the config-0 distributions (scale about 0.004) never reach."""
    import torch
    from turbo_fieldfare_b200.kernels import MPPPrefillInt4QMM
    o = oracle
    rng = np.random.default_rng(M + N)
    mat = o.quantize_rows(rng.uniform(-0.5, 0.5, size=(N, K)).astype(np.float32), 4)
    assert o.bf16_to_f32(mat.scales).min() > 2.0 ** -5
    x16 = o.f32_to_f16(rng.uniform(-1, 1, size=(M, K)).astype(np.float32))
    y = dev_zeros_u16(M * N, fill=0x7E00)
    assert MPPPrefillInt4QMM(tf_ctx).encode(to_dev(mat.packed), to_dev(mat.scales), to_dev(mat.biases), to_dev(x16), y, M, N, K) \
        == "affine-threadgroup-f16"
    torch.cuda.synchronize()
    _status_ok(tf_ctx)
    got = o.f16_to_f32(from_dev(y, np.uint16).reshape(M, N))
    ref = o.int4_qmm_ref(mat, x16)
    assert np.isfinite(got).all()
    assert o.rel_error(got, ref) <= QMM_TOL
    assert o.rel_l2(got, ref) <= QMM_TOL


def _route(rng, T, K, E, zipf):
    if zipf:
        p = 1.0 / (rng.permutation(E) + 1) ** 1.1
        p /= p.sum()
        return np.stack([rng.choice(E, size=K, replace=False, p=p) for _ in range(T)]).astype(np.uint32)
    return np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.uint32)


@pytest.mark.parametrize("T,D,F,E,K,zipf", [(5, 128, 64, 16, 8, False), (300, 256, 128, 8, 4, True),
                                            (256, 2816, 704, 16, 8, True)])
def test_grouped_tensorcore_vs_oracle_and_cuda_cores(tf_ctx, oracle, T, D, F, E, K, zipf):
    """Sorted-row tensor-core path == oracle per-pair partials == the CUDA-core grouped kernel, all within the
    chained-fp16 tolerance; groups of 1..>128 pairs exercise ragged token tiles."""
    import torch
    from turbo_fieldfare_b200.kernels import DeviceRoutes, PrefillGroupedRoutedMoE
    o = oracle
    rng = np.random.default_rng(T + D)
    off, payload, stride = o.blob_layout(D, F, align=256 if D < 2816 else 16384)
    pool_h = np.zeros(E * stride, dtype=np.uint8)
    for e in range(E):
        pool_h[e * stride:(e + 1) * stride] = random_blob(o, D, F, rng, off, stride)[0]
    h16 = o.f32_to_f16(rng.standard_normal((T, D)).astype(np.float32))
    idx = _route(rng, T, K, E, zipf)
    w16 = o.f32_to_f16(rng.dirichlet(np.ones(K), size=T).astype(np.float32))
    routes = DeviceRoutes(T, K, E)
    moe = PrefillGroupedRoutedMoE(tf_ctx)
    moe.encode_group_routes(to_dev(idx), to_dev(w16), T, K, E, routes)
    torch.cuda.synchronize()
    host = routes.to_host(T)
    tok = host.sorted_pairs["token"].astype(np.int64)
    rank = host.sorted_pairs["rank"].astype(np.int64)
    x_sorted = dev_zeros_u16(T * K * D)
    row_ids = torch.zeros(T * K, dtype=torch.int32, device="cuda")
    inverse = torch.zeros(T * K, dtype=torch.int32, device="cuda")
    moe.encode_pack_sorted_rows(to_dev(h16), routes, T, K, E, D, x_sorted, row_ids, inverse)
    torch.cuda.synchronize()
    # the pack stores every eight columns as (0,4,1,5,2,6,3,7) and records where each (token, rank) went
    packed = from_dev(x_sorted, np.uint16).reshape(T * K, D // 8, 8)
    assert np.array_equal(packed, h16[tok].reshape(T * K, D // 8, 8)[:, :, [0, 4, 1, 5, 2, 6, 3, 7]])
    assert np.array_equal(from_dev(row_ids, np.uint32), host.sorted_pairs["expert"])
    assert np.array_equal(from_dev(inverse, np.uint32).reshape(T, K)[tok, rank], np.arange(T * K))
    pool = to_dev(pool_h)
    acts = dev_zeros_u16(T * K * F)
    out_rows = dev_zeros_u16(T * K * D, fill=0x7E00)
    moe.encode_tensorcore(x_sorted, T * K, pool, stride, E, capi_offsets(off), routes, acts, out_rows, D, F)
    torch.cuda.synchronize()
    _status_ok(tf_ctx)
    got_sorted = o.f16_to_f32(from_dev(out_rows, np.uint16).reshape(T * K, D))
    got = np.zeros((T, K, D), dtype=np.float32)
    got[tok, rank] = got_sorted
    pairs = o.make_token_expert_pairs(idx, w16, T, K)
    ref = o.f16_to_f32(o.grouped_moe_pairs(pool_h, stride, off, h16, 0, pairs, D, F, K, T))
    assert np.isfinite(got).all()
    assert o.rel_l2(got, ref) < FP16_CHAINED
    assert o.rel_error(got, ref) < FP16_CHAINED
    partials = dev_zeros_u16(T * K * D, fill=0x7E00)
    acts2 = dev_zeros_u16(T * K * F)
    moe.encode_streamed_batched(to_dev(h16), pool, stride, capi_offsets(off), routes, acts2, partials, T, D, F, K)
    torch.cuda.synchronize()
    cores = o.f16_to_f32(from_dev(partials, np.uint16).reshape(T, K, D))
    assert o.rel_l2(got, cores) < FP16_CHAINED


@pytest.mark.parametrize("T,D,Fs", [(3, 128, 192), (130, 128, 192), (256, 2816, 2112)])
def test_shared_expert_tensorcore_vs_oracle(tf_ctx, oracle, T, D, Fs):
    import torch
    from turbo_fieldfare_b200.kernels import PrefillSharedExpert, SharedExpertProjection
    o = oracle
    rng = np.random.default_rng(99 + T)
    gate, up, down = config0_matrix(o, Fs, D, rng), config0_matrix(o, Fs, D, rng), config0_matrix(o, D, Fs, rng)
    x16 = o.f32_to_f16(rng.standard_normal((T, D)).astype(np.float32))
    proj = lambda m: SharedExpertProjection(to_dev(m.packed), to_dev(m.scales), to_dev(m.biases), m.m, m.n)
    y = dev_zeros_u16(T * D, fill=0x7E00)
    scratch = dev_zeros_u16(T * Fs)
    PrefillSharedExpert(tf_ctx).encode_block_tensorcore(to_dev(x16), proj(gate), proj(up), proj(down), y, scratch, T)
    torch.cuda.synchronize()
    _status_ok(tf_ctx)
    got = o.f16_to_f32(from_dev(y, np.uint16).reshape(T, D))
    assert np.isfinite(got).all()
    for t in sorted({0, T // 2, T - 1}):
        _, truth = o.shared_expert_int4(gate, up, down, x16[t], order=0)
        assert o.rel_l2(got[t], truth) < FP16_CHAINED
        assert o.rel_error(got[t], truth) < FP16_CHAINED
