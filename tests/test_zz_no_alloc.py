"""The allocation-free shared-expert entry point against the ordinary one.

``tf_shared_expert_int4_block_noalloc`` is for callers that may not allocate device memory (a server that gave all
HBM to its own pool at start-up, a plugin inside it, code running next to a graph capture). It keeps its activation
scratch in an array inside the library, shared by every call on the GPU, so this test calls it twice in a row with
different inputs and sizes: the second call finds the first call's activations in the array and must not care.
The file name sorts last so that the test also runs after every other test has used the GPU; it passes alone too.
"""
import ctypes as C

import numpy as np
import pytest

from helpers import config0_matrix, dev_zeros_u16, from_dev, to_dev

pytestmark = pytest.mark.gpu
FP16_CHAINED = 1e-2       # the tolerance of the other shared-expert tests


def _projection(m):
    from turbo_fieldfare_b200.kernels import SharedExpertProjection
    return SharedExpertProjection(to_dev(m.packed), to_dev(m.scales), to_dev(m.biases), m.m, m.n)


def test_noalloc_entry_matches_the_allocating_entry_twice_in_a_row(tf_ctx, oracle):
    import torch
    from turbo_fieldfare_b200 import _capi
    from turbo_fieldfare_b200.kernels import PrefillSharedExpert, _ptr
    o = oracle
    lib = _capi.load()
    rng = np.random.default_rng(4242)
    D, Fs = 256, 192
    gate, up, down = config0_matrix(o, Fs, D, rng), config0_matrix(o, Fs, D, rng), config0_matrix(o, D, Fs, rng)
    pg, pu, pd = _projection(gate), _projection(up), _projection(down)
    status_word = torch.full((1,), 7, dtype=torch.int32, device="cuda")       # the call must clear it
    for call, T in enumerate((40, 9)):                                          # second call: fewer rows, other data
        x16 = o.f32_to_f16(rng.standard_normal((T, D)).astype(np.float32) * (1.0 + call))
        x = to_dev(x16)
        # reference: the existing entry point with a caller-provided scratch
        y_ref = dev_zeros_u16(T * D, fill=0x7E00)
        scratch = dev_zeros_u16(T * Fs)
        PrefillSharedExpert(tf_ctx).encode_block(x, pg, pu, pd, y_ref, scratch, T)
        # under test: no context, no scratch
        y = dev_zeros_u16(T * D, fill=0x7E00)
        g, u, dn = pg.c_struct(), pu.c_struct(), pd.c_struct()
        st = lib.tf_shared_expert_int4_block_noalloc(None, _ptr(x), 0, D, C.byref(g), C.byref(u), C.byref(dn),
                                                     _ptr(y), 0, D, T, _ptr(status_word))
        assert st == 0, lib.tf_last_error(None).decode()
        torch.cuda.synchronize()
        assert int(status_word.item()) == 0
        got = o.f16_to_f32(from_dev(y, np.uint16).reshape(T, D))
        ref = o.f16_to_f32(from_dev(y_ref, np.uint16).reshape(T, D))
        assert np.isfinite(got).all()
        assert o.rel_l2(got, ref) < FP16_CHAINED
        assert o.rel_error(got, ref) < FP16_CHAINED
        # and both agree with the oracle on a row
        _, truth = o.shared_expert_int4(gate, up, down, x16[T - 1], order=0)
        assert o.rel_l2(got[T - 1], truth) < FP16_CHAINED


def test_noalloc_entry_rejects_blocks_beyond_its_scratch(tf_ctx):
    from turbo_fieldfare_b200 import _capi
    from turbo_fieldfare_b200._capi import Projection
    lib = _capi.load()
    p = Projection(None, 0, None, 0, None, 0, 2112, 2816)
    d = Projection(None, 0, None, 0, None, 0, 2816, 2112)
    st = lib.tf_shared_expert_int4_block_noalloc(None, None, 0, 2816, C.byref(p), C.byref(p), C.byref(d), None, 0, 2816, 249, None)
    assert st != 0
    msg = lib.tf_last_error(None).decode()
    assert "scratch" in msg and "tf_shared_expert_int4_block" in msg       # 249 * 2112 * 2 bytes > 1 MiB


def test_second_gpu_gets_its_own_kernel_attributes(oracle):
    """Kernel attributes (the raised shared-memory limit) belong to a device: after GPU 0 has run the kernels, both
    entry points must still work on GPU 1 in the same process. Needs two GPUs."""
    import torch
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from turbo_fieldfare_b200 import _capi
    from turbo_fieldfare_b200.kernels import PrefillSharedExpert, TurboContext, _ptr
    o = oracle
    lib = _capi.load()
    rng = np.random.default_rng(77)
    D, Fs, T = 2816, 2112, 12                 # production width: the kernels need more than 48 KB of shared memory
    gate, up, down = config0_matrix(o, Fs, D, rng), config0_matrix(o, Fs, D, rng), config0_matrix(o, D, Fs, rng)
    x16 = o.f32_to_f16(rng.standard_normal((T, D)).astype(np.float32))
    outs = []
    for device in (0, 1):
        torch.cuda.set_device(device)
        ctx = TurboContext(device)
        try:
            pg, pu, pd = _projection(gate), _projection(up), _projection(down)
            x = to_dev(x16)
            y_ref = dev_zeros_u16(T * D, fill=0x7E00)
            scratch = dev_zeros_u16(T * Fs)
            PrefillSharedExpert(ctx).encode_block(x, pg, pu, pd, y_ref, scratch, T)
            y = dev_zeros_u16(T * D, fill=0x7E00)
            g, u, dn = pg.c_struct(), pu.c_struct(), pd.c_struct()
            st = lib.tf_shared_expert_int4_block_noalloc(None, _ptr(x), 0, D, C.byref(g), C.byref(u), C.byref(dn),
                                                         _ptr(y), 0, D, T, None)
            assert st == 0, lib.tf_last_error(None).decode()
            torch.cuda.synchronize()
            assert ctx.device_status() == 0
            a, b = from_dev(y, np.uint16), from_dev(y_ref, np.uint16)
            assert np.array_equal(a, b)
            outs.append(a)
        finally:
            ctx.close()
            torch.cuda.set_device(0)
    assert np.array_equal(outs[0], outs[1])
