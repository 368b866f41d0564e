"""A `.gturbo` directory drives the MoE block unchanged: a synthetic install written to disk is opened, every
expert blob is copied to its logical slot of the HBM pool, the resident payload is uploaded, and the block
forward built from the checkpoint's tensor names matches the per-token oracle on the same bytes."""
import numpy as np
import pytest

from helpers import config0_matrix, from_dev, to_dev
from oracle import gturbo_writer as W

pytestmark = pytest.mark.gpu
TOL = 1e-2
D, F, FS, E, K, LAYERS = 128, 64, 128, 16, 8, 2


def _install(root, o, rng):
    table, payload = W.blob_tensor_table(D, F)
    off = o.ExpertOffsets(*[table[k]["offset"] for k in ("gate", "gate_scales", "gate_biases", "up", "up_scales",
                                                         "up_biases", "down", "down_scales", "down_biases")])
    experts, blobs, physical, resident, layers = [], [], [], [], []
    for L in range(LAYERS):
        mats = [(config0_matrix(o, F, D, rng), config0_matrix(o, F, D, rng), config0_matrix(o, D, F, rng)) for _ in range(E)]
        experts.append(mats)
        blobs.append([o.pack_blob(g, u, d, off, payload).tobytes() for g, u, d in mats])
        physical.append([int(v) for v in rng.permutation(E)])
        router = config0_matrix(o, E, D, rng, bits=8)
        scale = o.f32_to_bf16((1.0 + 0.25 * rng.standard_normal(D)).astype(np.float32))
        gain = o.f32_to_bf16((1.0 + 0.1 * rng.standard_normal(E)).astype(np.float32))
        sg, su, sd = config0_matrix(o, FS, D, rng), config0_matrix(o, FS, D, rng), config0_matrix(o, D, FS, rng)
        p = f"language_model.model.layers.{L}"

        def quantised(name, m, rows, cols_packed):
            w, s, b = W.affine_planes(m)
            return {"name": f"{p}.{name}", "dtype": W.DTYPE_U32, "shape": [rows, cols_packed, 0, 0],
                    "weights": w, "scales": s, "biases": b}
        resident += [
            quantised("router.proj.weight", router, E, D // 4),
            {"name": f"{p}.router.scale", "dtype": W.DTYPE_BF16, "shape": [D, 0, 0, 0], "weights": scale.tobytes()},
            {"name": f"{p}.router.per_expert_scale", "dtype": W.DTYPE_BF16, "shape": [E, 0, 0, 0], "weights": gain.tobytes()},
            quantised("mlp.gate_proj.weight", sg, FS, D // 8),
            quantised("mlp.up_proj.weight", su, FS, D // 8),
            quantised("mlp.down_proj.weight", sd, D, FS // 8),
        ]
        layers.append(dict(router=router, scale=scale, gain=gain, shared=(sg, su, sd)))
    meta = W.write_install(root, d=D, f=F, fs=FS, num_experts=E, top_k=K, blobs=blobs, physical_ranks=physical,
                           resident=resident)
    return meta, off, blobs, layers


def test_install_loads_into_hbm_and_runs_the_block(tf_ctx, oracle, tmp_path):
    import torch
    from turbo_fieldfare_b200.gturbo import GTurboDirectory, GTurboModel
    from turbo_fieldfare_b200.stack import Workspace, device_view_u8
    o = oracle
    rng = np.random.default_rng(2026)
    meta, off, blobs, layers = _install(tmp_path, o, rng)
    directory = GTurboDirectory.open(tmp_path)
    model = GTurboModel(tf_ctx, directory)
    assert model.layer_count == LAYERS

    # every blob sits at its LOGICAL slot, whatever its rank in the layer file
    for L in range(LAYERS):
        for e in range(E):
            got = device_view_u8(model.expert_ptr(L, e), meta["payload"]).cpu().numpy().tobytes()
            assert got == blobs[L][e], (L, e)

    T = 6
    x16 = o.f32_to_f16(rng.standard_normal((T, D)).astype(np.float32))
    ws = Workspace(tf_ctx, T, D, F, FS, K, E)
    for L in range(LAYERS):
        rec = model.layer(L)
        assert (rec.num_experts, rec.d, rec.f, rec.fs, rec.top_k, rec.expert_stride) == (E, D, F, FS, K, meta["stride"])
        # router.scale x 1/sqrt(D), rounded to bf16 (Runtime/Inference/RealForwardRunner.swift:352-376)
        eff = o.f32_to_bf16((o.bf16_to_f32(layers[L]["scale"]) * np.float32(1.0 / np.sqrt(np.float32(D)))).astype(np.float32))
        got_eff = device_view_u8(rec.effective_scale, 2 * D).cpu().numpy().view(np.uint16)
        assert np.array_equal(got_eff, eff)

        x, y = to_dev(x16.copy()), to_dev(np.zeros((T, D), np.uint16))
        model.block_forward(L, x, y, T, ws)
        torch.cuda.synchronize()
        assert tf_ctx.device_status() == 0
        got = o.f16_to_f32(from_dev(y, np.uint16).reshape(T, D))

        logits = o.router_logits(layers[L]["router"], x16, eff)
        idx, w16, _ = o.router_select(logits, layers[L]["gain"], K)
        got_idx, _ = ws.routing(T)
        assert np.array_equal(got_idx, idx)                  # routing is bit-exact
        sg, su, sd = layers[L]["shared"]
        ref = []
        for t in range(T):
            chosen = [np.frombuffer(blobs[L][int(e)], dtype=np.uint8) for e in idx[t]]
            shared16, _ = o.shared_expert_int4(sg, su, sd, x16[t], order=0)
            _, y32, _ = o.moe_routed_decode(chosen, off, x16[t], w16[t], shared16, D, F, order=0)
            ref.append(y32)
        assert o.rel_l2(got, np.stack(ref)) < TOL
    ws.close()
    model.close()
    directory.close()


def test_load_rejects_a_truncated_layer_file(tf_ctx, oracle, tmp_path):
    from turbo_fieldfare_b200.gturbo import GTurboDirectory, GTurboError, GTurboModel
    _install(tmp_path, oracle, np.random.default_rng(7))
    layer_file = tmp_path / "packed_experts" / "layer_01.bin"
    layer_file.write_bytes(layer_file.read_bytes()[:-4096])
    directory = GTurboDirectory.open(tmp_path)      # metadata is consistent; the payload is checked at load
    with pytest.raises(GTurboError) as err:
        GTurboModel(tf_ctx, directory)
    assert err.value.status == 201
    directory.close()
