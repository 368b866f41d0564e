"""GPU tests of the expert-parallel path: the pack kernel against the numpy plan, the single-rank EP
stack against the fused single-GPU stack, and (when two GPUs are visible) a 2-rank NCCL run against
the single-GPU result."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from helpers import from_dev, to_dev

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("T,capacity", [(5, 0), (64, 0), (64, 64 * 8), (1, 8)])
def test_pack_matches_numpy_plan(tf_ctx, oracle, T, capacity):
    import ctypes as C
    import torch
    from turbo_fieldfare_b200.ep import plan_dispatch
    from turbo_fieldfare_b200.kernels import DeviceRoutes, PrefillGroupedRoutedMoE
    K, E, D, world = 8, 128, 256, 4
    epr = E // world
    rng = np.random.default_rng(T + capacity)
    idx = np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.uint32)
    w16 = rng.integers(0, 0x3C00, size=(T, K)).astype(np.uint16)
    x16 = rng.integers(0, 0x7BFF, size=(T, D)).astype(np.uint16)
    routes = DeviceRoutes(T, K, E)
    PrefillGroupedRoutedMoE(tf_ctx).encode_group_routes(to_dev(idx), to_dev(w16), T, K, E, routes)
    slots = world * capacity if capacity else T * K
    # fixed-capacity rows carry the expert id in an 8-element tail (one exchange for rows and ids); exact rows are plain
    stride = D + 8 if capacity else D
    send_rows = torch.full((slots * stride,), -1, dtype=torch.int16, device="cuda")
    send_ids = torch.full((slots,), 7, dtype=torch.int32, device="cuda")
    inverse = torch.zeros(T * K, dtype=torch.int32, device="cuda")
    tf_ctx.check(tf_ctx.lib.tf_ep_pack(tf_ctx.handle, torch.cuda.current_stream().cuda_stream, to_dev(x16).data_ptr(), 0, D,
                                       C.byref(routes.c_struct), T, K, E, epr, capacity, D, send_rows.data_ptr(),
                                       send_ids.data_ptr(), inverse.data_ptr(), stride))
    torch.cuda.synchronize()
    assert tf_ctx.device_status() == 0
    tok, eloc, inv, _ = plan_dispatch(idx, epr, world, capacity)
    assert np.array_equal(from_dev(send_ids, np.uint32), eloc)
    assert np.array_equal(from_dev(inverse, np.uint32), inv)
    rows = from_dev(send_rows, np.uint16).reshape(slots, stride)
    valid = tok >= 0
    assert np.array_equal(rows[valid][:, :D], x16[tok[valid]])
    if capacity:
        tail_ids = np.ascontiguousarray(rows[:, D:D + 2]).view(np.uint32).reshape(slots)
        assert np.array_equal(tail_ids, eloc)
        ids2 = torch.zeros(slots, dtype=torch.int32, device="cuda")
        tf_ctx.check(tf_ctx.lib.tf_ep_extract_ids(tf_ctx.handle, torch.cuda.current_stream().cuda_stream, send_rows.data_ptr(),
                                                  stride, D, slots, ids2.data_ptr()))
        torch.cuda.synchronize()
        assert np.array_equal(from_dev(ids2, np.uint32), eloc)


def test_combine_and_reduce_take_more_rows_than_a_grid_dimension_holds(tf_ctx, oracle):
    """An expert-parallel rank whose experts are popular can hold more than 65535 rows (eight ranks, 4096 tokens each,
    a shard with twice the average traffic): the row count must not sit in a 16-bit grid dimension."""
    import torch
    o = oracle
    rows, D = 70001, 64
    rng = np.random.default_rng(70001)
    src = o.f32_to_f16(rng.standard_normal((rows, D)).astype(np.float32))
    perm = rng.permutation(rows).astype(np.uint32)
    ones = np.full(rows, 0x3C00, dtype=np.uint16)                 # fp16 1.0: an exact copy through the permutation
    st = torch.cuda.current_stream().cuda_stream
    out = torch.zeros(rows * D, dtype=torch.int16, device="cuda")
    d_src, d_ones, d_perm = to_dev(src), to_dev(ones), to_dev(perm)
    tf_ctx.check(tf_ctx.lib.tf_ep_combine(tf_ctx.handle, st, d_src.data_ptr(), d_ones.data_ptr(), d_perm.data_ptr(),
                                          None, D, out.data_ptr(), D, rows, 1, D))
    torch.cuda.synchronize()
    assert np.array_equal(from_dev(out, np.uint16).reshape(rows, D), src[perm])
    # the token-major reduce with one rank of weight 1.0 and fp16 partials rounds each value through fp32 and back
    out2 = torch.zeros(rows * D, dtype=torch.int16, device="cuda")
    tf_ctx.check(tf_ctx.lib.tf_moe_reduce_token_major(tf_ctx.handle, st, d_src.data_ptr(), 0, d_ones.data_ptr(), None, D,
                                                      out2.data_ptr(), D, rows, 1, D))
    torch.cuda.synchronize()
    assert np.array_equal(from_dev(out2, np.uint16).reshape(rows, D), src)


@pytest.mark.parametrize("T,fixed", [(1, True), (6, True), (70, False), (300, False)])   # 300 x 8 rows: tensor-core expert phase
def test_single_rank_ep_stack_matches_fused_stack(tf_ctx, oracle, T, fixed):
    import torch
    from turbo_fieldfare_b200.ep import ExpertParallelStack
    from turbo_fieldfare_b200.stack import MoEStack
    o = oracle
    dims = dict(layers=2, d=256, f=128, fs=192, num_experts=16, top_k=8, seed=5, align=256)
    ref_stack = MoEStack(tf_ctx, **dims)
    ep_stack = ExpertParallelStack(tf_ctx, **dims)
    rng = np.random.default_rng(T)
    h16 = o.f32_to_f16(rng.standard_normal((T, 256)).astype(np.float32))
    h_ref, h_ep = to_dev(h16.copy()), to_dev(h16.copy())
    ref_stack.forward(h_ref, T, ref_stack.workspace(T))
    ep_stack.forward(h_ep, T, ep_stack.buffers(T, fixed))
    torch.cuda.synchronize()
    assert tf_ctx.device_status() == 0
    a = o.f16_to_f32(from_dev(h_ref, np.uint16))
    b = o.f16_to_f32(from_dev(h_ep, np.uint16))
    # fp16 result rows over the wire instead of fp32 partials; at 300 tokens both stacks run tcgen05 GEMMs in different tilings
    assert o.rel_l2(b, a) < 3e-3
    ref_stack.close()
    ep_stack.close()


@pytest.mark.parametrize("T,fixed", [(1, True), (6, True), (70, False)])
def test_renumbered_experts_leave_the_outputs_alone(tf_ctx, oracle, T, fixed):
    """Experts placed by load: router rows and pool slots stored in another order. The measured load per ORIGINAL expert
    id and the stack's output must be those of the original numbering (one rank: the placement is the experts sorted
    by descending load, a non-trivial permutation)."""
    import torch
    from turbo_fieldfare_b200.ep import ExpertParallelStack, balanced_placement
    from turbo_fieldfare_b200.stack import MoEStack
    o = oracle
    dims = dict(layers=2, d=256, f=128, fs=192, num_experts=16, top_k=8, seed=5, align=256)
    ref_stack = MoEStack(tf_ctx, **dims)
    ep_stack = ExpertParallelStack(tf_ctx, **dims)
    rng = np.random.default_rng(900 + T)
    calib = to_dev(o.f32_to_f16(rng.standard_normal((40, 256)).astype(np.float32)))
    exact = ep_stack.buffers(40, False)
    load = ep_stack.expert_load(calib, 40, exact)
    assert load.shape == (2, 16) and np.all(load.sum(axis=1) == 40 * 8)
    placement = balanced_placement(tf_ctx.lib, load, 1)
    assert any(not np.array_equal(placement[l], np.arange(16)) for l in range(2))
    ep_stack.set_placement(placement)
    assert np.array_equal(ep_stack.expert_load(calib, 40, exact), load)
    h16 = o.f32_to_f16(rng.standard_normal((T, 256)).astype(np.float32))
    h_ref, h_ep = to_dev(h16.copy()), to_dev(h16.copy())
    ref_stack.forward(h_ref, T, ref_stack.workspace(T))
    ep_stack.forward(h_ep, T, ep_stack.buffers(T, fixed))
    torch.cuda.synchronize()
    assert tf_ctx.device_status() == 0
    a = o.f16_to_f32(from_dev(h_ref, np.uint16))
    b = o.f16_to_f32(from_dev(h_ep, np.uint16))
    assert o.rel_l2(b, a) < 3e-3
    # back to the original numbering: the contiguous stack again
    ep_stack.set_placement(None)
    h_back = to_dev(h16.copy())
    ep_stack.forward(h_back, T, ep_stack.buffers(T, fixed))
    torch.cuda.synchronize()
    assert o.rel_l2(o.f16_to_f32(from_dev(h_back, np.uint16)), a) < 3e-3
    ref_stack.close()
    ep_stack.close()


@pytest.mark.parametrize("T,tensor_rows", [(1, 0), (6, 0), (64, 0), (6, 1), (64, 1), (64, 100000)])
def test_single_rank_peer_exchange_matches_fused_stack_and_replays_in_a_graph(tf_ctx, oracle, T, tensor_rows):
    """The peer-memory exchange with one rank (the rank pushes into its own buffer and passes its own flag barrier):
    same result as the fused stack, eagerly and as a replayed CUDA graph of the whole step. tensor_rows = 1 forces the
    owner's expert phase onto the tensor cores (most slots of the fixed-capacity buffer are empty then), 100000 onto
    the streaming kernels, 0 leaves the library's default (streaming kernels)."""
    import torch
    from turbo_fieldfare_b200.ep import ExpertParallelStack
    from turbo_fieldfare_b200.stack import MoEStack
    o = oracle
    tf_ctx.set_ep_tensorcore_min_rows_per_expert(tensor_rows or 0xFFFFFFFF)
    dims = dict(layers=2, d=256, f=128, fs=192, num_experts=16, top_k=8, seed=5, align=256)
    ref_stack = MoEStack(tf_ctx, **dims)
    ep_stack = ExpertParallelStack(tf_ctx, **dims)
    rng = np.random.default_rng(40 + T)
    h16 = o.f32_to_f16(rng.standard_normal((T, 256)).astype(np.float32))
    h_ref = to_dev(h16.copy())
    ref_stack.forward(h_ref, T, ref_stack.workspace(T))
    want = o.f16_to_f32(from_dev(h_ref, np.uint16))
    buf = ep_stack.buffers(T, True, peer=True)
    h_ep = to_dev(h16.copy())
    ep_stack.forward(h_ep, T, buf)
    torch.cuda.synchronize()
    assert tf_ctx.device_status() == 0
    assert o.rel_l2(o.f16_to_f32(from_dev(h_ep, np.uint16)), want) < 3e-3
    # the same step as a graph, replayed twice on fresh inputs
    static_h = to_dev(h16.copy())
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ep_stack.forward(static_h, T, buf)          # warm-up on the capture stream
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ep_stack.forward(static_h, T, buf)
    for _ in range(2):
        static_h.copy_(to_dev(h16.copy()))
        graph.replay()
        torch.cuda.synchronize()
        assert o.rel_l2(o.f16_to_f32(from_dev(static_h, np.uint16)), want) < 3e-3
    assert tf_ctx.device_status() == 0
    tf_ctx.set_ep_tensorcore_min_rows_per_expert(0xFFFFFFFF)
    buf.close()
    ref_stack.close()
    ep_stack.close()


def test_peer_barrier_wait_runs_out_and_reports(oracle):
    """A barrier whose second participant never arrives (its flag is a word that nothing sets): the bounded wait gives
    up after about two seconds, the kernel returns, the context reports the device code and stays usable, and a later
    barrier passes. No fault, no hang: the wait simply runs out."""
    import ctypes as C
    import time
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from turbo_fieldfare_b200.kernels import TFError, TurboContext
    ctx = TurboContext(0)
    lib = ctx.lib
    handle = C.c_void_p()
    ctx.check(lib.tf_peer_buffer_create(ctx.handle, 4096, C.byref(handle)))
    own = lib.tf_peer_buffer_ptr(handle)
    # "world" of two whose second member is this same buffer, 1 KiB further on: rank 0 signals it and then waits for
    # flag word 1 of its own buffer, which nobody writes
    bases = torch.tensor([own, own + 1024], dtype=torch.int64, device="cuda")
    epoch = torch.zeros(2, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    t0 = time.time()
    ctx.check(lib.tf_ep_peer_barrier(ctx.handle, st, bases.data_ptr(), 0, epoch.data_ptr(), 2, 0))
    with pytest.raises(TFError) as err:
        ctx.device_status()
    waited = time.time() - t0
    assert "0x7f000011" in str(err.value).lower()
    assert waited < 30.0
    # the context is still usable: a one-member barrier passes and the status is clean again
    ctx.check(lib.tf_ep_peer_barrier(ctx.handle, st, bases.data_ptr(), 0, epoch.data_ptr(), 1, 0))
    assert ctx.device_status() == 0
    assert int(epoch.cpu()[0]) == 2
    lib.tf_peer_buffer_destroy(handle)
    ctx.close()


def test_two_rank_nccl_matches_single_gpu(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(ROOT / "tests" / "ep_rank_main.py"), str(tmp_path)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    errs = [float(np.load(tmp_path / f"err_{r}.npy")) for r in range(2)]
    assert max(errs) < 3e-3, errs
