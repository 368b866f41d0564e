"""GPU parity of the fused MoE block and the layer stack against the oracle applied per token
(benchmark configurations 1 and 2, and a small-dimension stack)."""
import numpy as np
import pytest

from helpers import from_dev, to_dev

pytestmark = pytest.mark.gpu
TOL = 1e-2     # benchmark bound: outputs within 1e-2 relative L2 of the fp32-dequantised oracle


def _affine_from(o, tensor):
    packed, scales, biases = tensor.download()
    return o.AffineMatrix(packed, scales, biases, tensor.bits, tensor.cols)


def _oracle_offsets(o, coff):
    return o.ExpertOffsets(coff.gate_w_off, coff.gate_s_off, coff.gate_b_off, coff.up_w_off, coff.up_s_off,
                           coff.up_b_off, coff.down_w_off, coff.down_s_off, coff.down_b_off)


def _oracle_block(o, layer, pool, x16_rows, tokens, logit_bias=None):
    """Per-token oracle of one block. Returns (indices, y_f32 [T, D], w_f32)."""
    router = _affine_from(o, layer.router)
    sg, su, sd = (_affine_from(o, t) for t in (layer.shared_gate, layer.shared_up, layer.shared_down))
    eff = from_dev(layer.effective_scale, np.uint16)
    gain = from_dev(layer.per_expert_scale, np.uint16)
    logits = o.router_logits(router, x16_rows, eff)
    if logit_bias is not None:
        logits = (logits + logit_bias.astype(np.float32)).astype(np.float32)
    idx, w16, w32 = o.router_select(logits, gain, layer.top_k)
    off = _oracle_offsets(o, pool.offsets)
    cache = {}
    ys = []
    for t in tokens:
        blobs = []
        for e in idx[t]:
            if int(e) not in cache:
                cache[int(e)] = pool.download(layer.layer_index, int(e))
            blobs.append(cache[int(e)])
        shared16, _ = o.shared_expert_int4(sg, su, sd, x16_rows[t], order=0)
        _, y32, _ = o.moe_routed_decode(blobs, off, x16_rows[t], w16[t], shared16, layer.d, layer.f, order=0)
        ys.append(y32)
    return idx, (np.stack(ys) if ys else np.zeros((0, layer.d), np.float32)), w32


@pytest.fixture(scope="module")
def production_layer(tf_ctx):
    """One production-shaped layer: 128 experts of the .gturbo blob layout (430 MB)."""
    import torch
    from turbo_fieldfare_b200.stack import ExpertPool, MoEBlockLayer
    pool = ExpertPool(tf_ctx, 1, 128, 2816, 704)
    assert pool.stride == 3358720 and pool.nbytes == 429916160      # docs/SYSTEM_DESIGN.md:166
    pool.fill_synthetic(11)
    layer = MoEBlockLayer(tf_ctx, pool, 0, 2816, 704, 2112, 128, 8)
    layer.fill_synthetic(12)
    torch.cuda.synchronize()
    yield layer, pool
    pool.close()


def test_synthetic_weights_follow_the_config_distributions(tf_ctx, oracle, production_layer):
    o = oracle
    layer, pool = production_layer
    blob = pool.download(0, 5)
    off = pool.offsets
    codes = blob[off.gate_w_off:off.gate_w_off + 704 * 1408]
    nib = np.concatenate([codes & 0xF, codes >> 4])
    hist = np.bincount(nib, minlength=16) / nib.size
    assert np.all(np.abs(hist - 1 / 16) < 0.002)                      # uniform 0..15
    s = o.bf16_to_f32(blob[off.gate_s_off:off.gate_s_off + 704 * 44 * 2].view(np.uint16))
    b = o.bf16_to_f32(blob[off.gate_b_off:off.gate_b_off + 704 * 44 * 2].view(np.uint16))
    assert abs(s.mean() - 0.004 * np.sqrt(2 / np.pi)) < 2e-4 and s.min() >= 0      # |N(0,1)| * 0.004
    assert np.abs(b + 8 * s).max() < 1e-3 + 8 * s.max() * 2 ** -8                # -8 * scale + N(0, 1e-4), bf16
    assert np.any(blob[off.down_w_off:off.down_w_off + 64] != 0) and np.all(blob[pool.payload:] == 0)
    other = pool.download(0, 6)
    assert not np.array_equal(other[:4096], blob[:4096])


@pytest.mark.parametrize("T", [1, 64])
def test_block_forward_configs_1_and_2(tf_ctx, oracle, production_layer, T):
    """Config 1 (one token) and config 2 (64 tokens): top-k indices bit-exact, outputs within tolerance."""
    import torch
    from turbo_fieldfare_b200.stack import MoEBlock, Workspace
    o = oracle
    layer, pool = production_layer
    rng = np.random.default_rng(100 + T)
    x16 = o.f32_to_f16(rng.standard_normal((T, 2816)).astype(np.float32))
    ws = Workspace(tf_ctx, T, 2816, 704, 2112, 8, 128)
    y = torch.zeros(T * 2816, dtype=torch.int16, device="cuda")
    launches0 = tf_ctx.launch_count
    MoEBlock(tf_ctx, layer).forward(to_dev(x16), y, T, ws)
    torch.cuda.synchronize()
    assert tf_ctx.launch_count - launches0 == 6     # router+grouping, gate/up, down, 2 x shared expert, combine
    idx_gpu, w_gpu = ws.routing(T)
    check = range(T) if T == 1 else (0, 13, 63)
    idx_ref, y_ref, w_ref = _oracle_block(o, layer, pool, x16, check)
    assert np.array_equal(idx_gpu, idx_ref), "top-k indices differ from the oracle"
    assert np.max(np.abs(o.f16_to_f32(w_gpu) - w_ref)) < 5e-3
    got = o.f16_to_f32(from_dev(y, np.uint16).reshape(T, 2816))
    for i, t in enumerate(check):
        assert o.rel_l2(got[t], y_ref[i]) < TOL, f"token {t}"
    if T == 64:
        counts = np.bincount(idx_gpu.reshape(-1), minlength=128)
        assert counts.sum() == 512 and (counts > 0).sum() > 100        # near-uniform load touches most experts


def test_block_forward_with_zipf_bias_and_fp16_partials(tf_ctx, oracle, production_layer):
    """Config-3 routing skew at a test-sized token count; workspace > 64 tokens selects fp16 partials."""
    import torch
    from turbo_fieldfare_b200.stack import MoEBlock, Workspace
    o = oracle
    layer, pool = production_layer
    rng = np.random.default_rng(7)
    T = 96
    p = 1.0 / (rng.permutation(128) + 1) ** 1.1
    bias = np.log(p / p.sum()).astype(np.float32)
    layer.set_logit_bias(bias)
    try:
        x16 = o.f32_to_f16(rng.standard_normal((T, 2816)).astype(np.float32))
        ws = Workspace(tf_ctx, 128, 2816, 704, 2112, 8, 128)
        y = torch.zeros(T * 2816, dtype=torch.int16, device="cuda")
        MoEBlock(tf_ctx, layer).forward(to_dev(x16), y, T, ws)
        torch.cuda.synchronize()
        idx_gpu, _ = ws.routing(T)
        check = (0, 50, 95)
        idx_ref, y_ref, _ = _oracle_block(o, layer, pool, x16, check, logit_bias=bias)
        assert np.array_equal(idx_gpu, idx_ref)
        got = o.f16_to_f32(from_dev(y, np.uint16).reshape(T, 2816))
        for i, t in enumerate(check):
            assert o.rel_l2(got[t], y_ref[i]) < TOL
        counts = np.bincount(idx_gpu.reshape(-1), minlength=128)
        assert counts.max() > 4 * counts.mean()                          # the skew is real
    finally:
        layer.set_logit_bias(None)


def _sample_rows(idx_ref, T, n_random, seed):
    """Rows worth checking on a tiled path: the first and last row of the hottest expert's group (its last, ragged
    128-token tile), the row of a one-row group if there is one, the block's first and last row, plus a seeded
    random sample."""
    counts = np.bincount(idx_ref.reshape(-1), minlength=int(idx_ref.max()) + 1)
    rows = {0, T - 1}
    hot = int(np.argmax(counts))
    hot_rows = np.nonzero((idx_ref == hot).any(axis=1))[0]
    rows.update((int(hot_rows[0]), int(hot_rows[-1])))
    ones = np.nonzero(counts == 1)[0]
    if ones.size:
        rows.add(int(np.nonzero((idx_ref == ones[0]).any(axis=1))[0][0]))
    rng = np.random.default_rng(seed)
    rows.update(int(r) for r in rng.choice(T, size=min(n_random, T), replace=False))
    return sorted(rows)


@pytest.mark.parametrize("T,zipf", [(256, False), (1000, True), (4096, True)])
def test_block_forward_prefill_sized_runs_on_tensor_cores(tf_ctx, oracle, production_layer, T, zipf):
    """From 256 tokens the block runs pack -> tcgen05 grouped GEMMs -> combine; same router decisions on EVERY row,
    outputs within the same 1e-2 relative L2 of the per-token oracle on at least 32 rows. T = 4096 with the
    Zipf(1.1) logit bias is benchmark configuration 3 on one GPU."""
    import torch
    from turbo_fieldfare_b200.stack import MoEBlock, Workspace
    o = oracle
    layer, pool = production_layer
    rng = np.random.default_rng(70 + T)
    bias = None
    if zipf:
        p = 1.0 / (rng.permutation(128) + 1) ** 1.1
        bias = np.log(p / p.sum()).astype(np.float32)
    layer.set_logit_bias(bias)
    try:
        x16 = o.f32_to_f16(rng.standard_normal((T, 2816)).astype(np.float32))
        ws = Workspace(tf_ctx, T, 2816, 704, 2112, 8, 128)
        y = torch.zeros(T * 2816, dtype=torch.int16, device="cuda")
        before = tf_ctx.launch_count
        MoEBlock(tf_ctx, layer).forward(to_dev(x16), y, T, ws)
        torch.cuda.synchronize()
        assert tf_ctx.device_status() == 0
        # router (two launches), grouping (three launches from 4096 pairs on), pack, 3 x (prepare + GEMM) ... combine
        assert tf_ctx.launch_count - before == (15 if T * 8 >= 4096 else 13)
        idx_gpu, w_gpu = ws.routing(T)
        idx_all, _, w_all = _oracle_block(o, layer, pool, x16, (), logit_bias=bias)
        assert np.array_equal(idx_gpu, idx_all), "top-k indices differ from the oracle on some row"
        assert np.max(np.abs(o.f16_to_f32(w_gpu) - w_all)) < 5e-3
        if zipf:
            counts = np.bincount(idx_all.reshape(-1), minlength=128)
            assert counts.max() > 4 * counts.mean()
        check = _sample_rows(idx_all, T, 32, T)
        assert len(check) >= 32
        _, y_ref, _ = _oracle_block(o, layer, pool, x16, check, logit_bias=bias)
        got = o.f16_to_f32(from_dev(y, np.uint16).reshape(T, 2816))
        assert np.isfinite(got).all()
        for i, t in enumerate(check):
            assert o.rel_l2(got[t], y_ref[i]) < TOL, f"token {t}"
    finally:
        layer.set_logit_bias(None)


@pytest.mark.parametrize("T", [5, 4096])
def test_block_forward_bf16_rows(tf_ctx, oracle, production_layer, T):
    """benchmark configuration 3 names bf16 activations: the block takes bf16 rows, converts them to fp16 exactly (every bf16
    value of normalised activations is an fp16 value), and rounds its result to bf16. Same router decisions as the oracle
    on every row; outputs within 1e-2 relative L2 plus the bf16 rounding of the result (2^-9)."""
    import torch
    from turbo_fieldfare_b200.stack import MoEBlock, Workspace
    o = oracle
    layer, pool = production_layer
    rng = np.random.default_rng(300 + T)
    p = 1.0 / (rng.permutation(128) + 1) ** 1.1
    bias = np.log(p / p.sum()).astype(np.float32)
    layer.set_logit_bias(bias)
    try:
        xb = o.f32_to_bf16(rng.standard_normal((T, 2816)).astype(np.float32))
        x16 = o.f32_to_f16(o.bf16_to_f32(xb))
        xf = o.bf16_to_f32(xb)
        normal = np.abs(xf) >= 2.0 ** -14
        assert np.array_equal(o.f16_to_f32(x16)[normal], xf[normal])             # exact inside fp16's normal range
        assert np.max(np.abs(o.f16_to_f32(x16) - xf)) <= 2.0 ** -25              # below it: fp16's subnormal spacing
        ws = Workspace(tf_ctx, T, 2816, 704, 2112, 8, 128)
        y = torch.zeros(T * 2816, dtype=torch.int16, device="cuda")
        MoEBlock(tf_ctx, layer).forward_bf16(to_dev(xb), y, T, ws)
        torch.cuda.synchronize()
        assert tf_ctx.device_status() == 0
        idx_gpu, _ = ws.routing(T)
        idx_all, _, _ = _oracle_block(o, layer, pool, x16, (), logit_bias=bias)
        assert np.array_equal(idx_gpu, idx_all), "top-k indices differ from the oracle on some row"
        check = _sample_rows(idx_all, T, 16, T)
        _, y_ref, _ = _oracle_block(o, layer, pool, x16, check, logit_bias=bias)
        got = o.bf16_to_f32(from_dev(y, np.uint16).reshape(T, 2816))
        assert np.isfinite(got).all()
        for i, t in enumerate(check):
            assert o.rel_l2(got[t], y_ref[i]) < TOL + 2.0 ** -8, f"token {t}"
    finally:
        layer.set_logit_bias(None)


def test_small_stack_matches_oracle(tf_ctx, oracle):
    """Config-4 structure at small dimensions: 3 layers, RMSNorm between layers, residual stream."""
    import torch
    from turbo_fieldfare_b200.stack import MoEStack
    o = oracle
    stack = MoEStack(tf_ctx, layers=3, d=256, f=128, fs=192, num_experts=16, top_k=8, seed=5, align=256)
    T = 4
    rng = np.random.default_rng(9)
    h16 = o.f32_to_f16(rng.standard_normal((T, 256)).astype(np.float32))
    hid = to_dev(h16.copy())
    ws = stack.workspace(T)
    stack.forward(hid, T, ws)
    torch.cuda.synchronize()
    got = o.f16_to_f32(from_dev(hid, np.uint16).reshape(T, 256))
    # oracle: same recurrence with fp16 rounding at the same points
    h = h16.copy()
    for l, layer in enumerate(stack.layers):
        x = o.rmsnorm(h, from_dev(stack.norm_weights[l], np.uint16))
        _, y32, _ = _oracle_block(o, layer, stack.pool, x, range(T))
        y16 = o.f32_to_f16(y32)
        h = o.f32_to_f16(o.f16_to_f32(h) + o.f16_to_f32(y16))
    ref = o.f16_to_f32(h)
    assert o.rel_l2(got, ref) < TOL
    stack.close()


@pytest.mark.parametrize("T,single_launch", [(1, False), (1, True), (8, False), (64, False), (300, False)])
def test_production_width_stack_matches_oracle(tf_ctx, oracle, T, single_launch):
    """Config-4 structure at production width (D = 2816, 128 experts, top-8, Fs = 2112), two layers: one token (layer
    by layer and as the single-launch decode step), decode batches and a tensor-core sized block against the
    per-token oracle recurrence."""
    import torch
    from turbo_fieldfare_b200.stack import MoEStack
    o = oracle
    stack = MoEStack(tf_ctx, layers=2, seed=31)
    tf_ctx.set_single_launch_step(single_launch)
    try:
        rng = np.random.default_rng(400 + T)
        h16 = o.f32_to_f16(rng.standard_normal((T, 2816)).astype(np.float32))
        hid = to_dev(h16.copy())
        ws = stack.workspace(T)
        stack.forward(hid, T, ws)
        torch.cuda.synchronize()
        assert tf_ctx.device_status() == 0
        got = o.f16_to_f32(from_dev(hid, np.uint16).reshape(T, 2816))
        rows = sorted({0, T - 1} | {int(r) for r in rng.choice(T, size=min(T, 6), replace=False)})
        h = h16[rows].copy()
        for l, layer in enumerate(stack.layers):
            h_before_last = h.copy()
            x = o.rmsnorm(h, from_dev(stack.norm_weights[l], np.uint16))
            _, y32, _ = _oracle_block(o, layer, stack.pool, x, range(len(rows)))
            h = o.f32_to_f16(o.f16_to_f32(h) + o.f16_to_f32(o.f32_to_f16(y32)))
        ref = o.f16_to_f32(h)
        assert np.isfinite(got).all()
        for i, t in enumerate(rows):
            assert o.rel_l2(got[t], ref[i]) < TOL, f"token {t}"
        if single_launch:
            # the step's last router decision equals the oracle's for the last layer's input
            idx_gpu, _ = ws.routing(1)
            x_last = o.rmsnorm(h_before_last, from_dev(stack.norm_weights[-1], np.uint16))
            idx_ref, _, _ = _oracle_block(o, stack.layers[-1], stack.pool, x_last, ())
            assert np.array_equal(idx_gpu, idx_ref[:1])
    finally:
        tf_ctx.set_single_launch_step(False)
        stack.close()


def test_one_token_stack_equals_layered_path(tf_ctx, oracle):
    """The one-token decode step of the stack against the same layers run block by block through
    tf_residual_rmsnorm + tf_moe_block_forward: same router decisions, outputs within fp16 rounding of each other."""
    import ctypes as C
    import torch
    from turbo_fieldfare_b200.kernels import _ptr
    from turbo_fieldfare_b200.stack import MoEBlock, MoEStack
    o = oracle
    stack = MoEStack(tf_ctx, layers=3, d=256, f=128, fs=192, num_experts=16, top_k=8, seed=5, align=256)
    try:
        rng = np.random.default_rng(3)
        h16 = o.f32_to_f16(rng.standard_normal((1, 256)).astype(np.float32))
        hid = to_dev(h16.copy())
        ws = stack.workspace(1)
        tf_ctx.set_single_launch_step(True)
        before = tf_ctx.launch_count
        stack.forward(hid, 1, ws)
        torch.cuda.synchronize()
        tf_ctx.set_single_launch_step(False)
        assert tf_ctx.launch_count - before == 1
        assert tf_ctx.device_status() == 0
        got = o.f16_to_f32(from_dev(hid, np.uint16))
        # block by block
        lib = tf_ctx.lib
        hid2 = to_dev(h16.copy())
        x = torch.zeros(256, dtype=torch.int16, device="cuda")
        y = torch.zeros(256, dtype=torch.int16, device="cuda")
        ws2 = stack.workspace(1)
        y_prev = None
        for l, layer in enumerate(stack.layers):
            tf_ctx.check(lib.tf_residual_rmsnorm(tf_ctx.handle, 0, _ptr(hid2), _ptr(y_prev), _ptr(stack.norm_weights[l]), _ptr(x), 1, 256,
                                                 C.c_float(1e-6)))
            MoEBlock(tf_ctx, layer).forward(x, y, 1, ws2, stream=0)
            y_prev = y
        tf_ctx.check(lib.tf_residual_rmsnorm(tf_ctx.handle, 0, _ptr(hid2), _ptr(y_prev), None, None, 1, 256, C.c_float(1e-6)))
        torch.cuda.synchronize()
        ref_bits = from_dev(hid2, np.uint16)
        ref = o.f16_to_f32(ref_bits)
        assert o.rel_l2(got, ref) < 2e-3
        # the layered stack forward folds each layer's reduce into the next norm: same bits as the chain of entry points
        hid3 = to_dev(h16.copy())
        stack.forward(hid3, 1, stack.workspace(1))
        torch.cuda.synchronize()
        assert np.array_equal(from_dev(hid3, np.uint16), ref_bits)
    finally:
        stack.close()


@pytest.mark.parametrize("T,d", [(7, 256), (40, 2816)])
def test_decode_sized_stack_equals_the_chain_of_entry_points_bit_for_bit(tf_ctx, oracle, T, d):
    """tf_stack_forward on a decode-sized batch forms the weighted sum of the route partials inside the next norm; the
    hidden state must equal tf_residual_rmsnorm + tf_moe_block_forward layer by layer, bit for bit (d = 2816: three
    slices of the norm's sum of squares, the last one partial)."""
    import ctypes as C
    import torch
    from turbo_fieldfare_b200.kernels import _ptr
    from turbo_fieldfare_b200.stack import MoEBlock, MoEStack
    o = oracle
    dims = dict(layers=3, d=d, f=128, fs=192, num_experts=16, top_k=8, seed=11, align=256)
    stack = MoEStack(tf_ctx, **dims)
    try:
        rng = np.random.default_rng(T + d)
        h16 = o.f32_to_f16(rng.standard_normal((T, d)).astype(np.float32))
        a = to_dev(h16.copy())
        stack.forward(a, T, stack.workspace(T))
        lib = tf_ctx.lib
        b = to_dev(h16.copy())
        x = torch.zeros(T * d, dtype=torch.int16, device="cuda")
        y = torch.zeros(T * d, dtype=torch.int16, device="cuda")
        ws = stack.workspace(T)
        y_prev = None
        for l, layer in enumerate(stack.layers):
            tf_ctx.check(lib.tf_residual_rmsnorm(tf_ctx.handle, 0, _ptr(b), _ptr(y_prev), _ptr(stack.norm_weights[l]), _ptr(x), T, d,
                                                 C.c_float(1e-6)))
            MoEBlock(tf_ctx, layer).forward(x, y, T, ws, stream=0)
            y_prev = y
        tf_ctx.check(lib.tf_residual_rmsnorm(tf_ctx.handle, 0, _ptr(b), _ptr(y_prev), None, None, T, d, C.c_float(1e-6)))
        torch.cuda.synchronize()
        assert tf_ctx.device_status() == 0
        assert np.array_equal(from_dev(a, np.uint16), from_dev(b, np.uint16))
    finally:
        stack.close()


@pytest.mark.parametrize("T", [1, 40])
def test_block_forward_with_8bit_shared_expert(tf_ctx, oracle, T):
    """A layer whose shared expert is 8-bit affine (tf_moe_layer.shared_bits = 8; SharedExpertInt8.swift:55-210): the
    block runs the fused 8-bit gate/up + down beside the routed experts."""
    import torch
    from turbo_fieldfare_b200.stack import ExpertPool, MoEBlock, MoEBlockLayer, Workspace
    o = oracle
    d, f, fs, E, K = 256, 128, 192, 16, 8
    pool = ExpertPool(tf_ctx, 1, E, d, f, align=256)
    pool.fill_synthetic(21)
    layer = MoEBlockLayer(tf_ctx, pool, 0, d, f, fs, E, K, shared_bits=8)
    layer.fill_synthetic(22)
    try:
        rng = np.random.default_rng(T)
        x16 = o.f32_to_f16(rng.standard_normal((T, d)).astype(np.float32))
        ws = Workspace(tf_ctx, T, d, f, fs, K, E)
        y = torch.zeros(T * d, dtype=torch.int16, device="cuda")
        MoEBlock(tf_ctx, layer).forward(to_dev(x16), y, T, ws)
        torch.cuda.synchronize()
        assert tf_ctx.device_status() == 0
        router = _affine_from(o, layer.router)
        sg, su, sd = (_affine_from(o, t) for t in (layer.shared_gate, layer.shared_up, layer.shared_down))
        assert sg.bits == 8
        eff = from_dev(layer.effective_scale, np.uint16)
        gain = from_dev(layer.per_expert_scale, np.uint16)
        idx_ref, w16, _ = o.router_select(o.router_logits(router, x16, eff), gain, K)
        idx_gpu, _ = ws.routing(T)
        assert np.array_equal(idx_gpu, idx_ref)
        off = _oracle_offsets(o, pool.offsets)
        got = o.f16_to_f32(from_dev(y, np.uint16).reshape(T, d))
        for t in sorted({0, T // 2, T - 1}):
            x = o.f16_to_f32(x16[t])
            g, u = o.gemv_ref(sg, x), o.gemv_ref(su, x)
            g, u = o.f16_to_f32(o.f32_to_f16(g)), o.f16_to_f32(o.f32_to_f16(u))
            inner = np.clip(0.7978845608028654 * (g.astype(np.float64) + 0.044715 * g.astype(np.float64) ** 3), -20, 20)
            act = o.f32_to_f16((0.5 * g * (1.0 + np.tanh(inner))).astype(np.float32) * u)
            shared16 = o.f32_to_f16(o.gemv_ref(sd, o.f16_to_f32(act)))
            blobs = [pool.download(0, int(e)) for e in idx_ref[t]]
            _, ref, _ = o.moe_routed_decode(blobs, off, x16[t], w16[t], shared16, d, f, order=0)
            assert o.rel_l2(got[t], ref) < TOL, f"token {t}"
    finally:
        pool.close()
