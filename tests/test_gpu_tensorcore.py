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


def test_int4_qmm_rejects_bad_k(tf_ctx):
    from turbo_fieldfare_b200.kernels import MPPPrefillInt4QMM, TFError
    z = dev_zeros_u16(64 * 64)
    with pytest.raises(TFError):
        MPPPrefillInt4QMM(tf_ctx).encode(z, z, z, z, z, 4, 64, 96)      # K % 64 != 0 (MPPPrefillInt4QMM.swift:43-55)


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
