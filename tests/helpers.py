"""Shared fixtures-as-functions for the parity tests: seeded inputs (the
reference's PRNG and quantisers through the oracle, or numpy for the benchmark
configurations) and upload helpers. Test infrastructure only."""
from __future__ import annotations

import numpy as np


def to_dev(a: np.ndarray):
    import torch
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).cuda()
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).cuda()
    if a.dtype == np.uint64:
        return torch.from_numpy(a.view(np.int64)).cuda()
    return torch.from_numpy(a).cuda()


def from_dev(t, dtype):
    return t.detach().cpu().numpy().view(dtype)


def dev_zeros_u16(n, fill=0):
    import torch
    t = torch.full((n,), 0, dtype=torch.int16, device="cuda")
    if fill:
        t.fill_(np.array(fill, dtype=np.uint16).view(np.int16).item())
    return t


def config0_matrix(o, m, n, rng, sb_dtype=0, bits=4):
    """benchmark configuration-0 distributions: uniform codes, scale=|N(0,1)|*0.004,
    bias=-8*scale+N(0,1e-4) (1e-4 read as the standard deviation), both rounded to the
    16-bit plane dtype; for 8-bit codes the recipe is scaled (scale/16, bias=-128*scale)."""
    if bits == 4:
        codes = rng.integers(0, 16, size=(m, n), dtype=np.uint8)
        packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
        scale = np.abs(rng.standard_normal((m, n // 64))).astype(np.float32) * np.float32(0.004)
        bias = (-8.0 * scale + rng.standard_normal((m, n // 64)).astype(np.float32) * np.float32(1e-4)).astype(np.float32)
    else:
        packed = rng.integers(0, 256, size=(m, n), dtype=np.uint8)
        scale = np.abs(rng.standard_normal((m, n // 64))).astype(np.float32) * np.float32(0.004 / 16)
        bias = (-128.0 * scale + rng.standard_normal((m, n // 64)).astype(np.float32) * np.float32(1e-4)).astype(np.float32)
    conv = o.f32_to_bf16 if sb_dtype == 0 else o.f32_to_f16
    return o.AffineMatrix(np.ascontiguousarray(packed), conv(scale), conv(bias), bits, n, sb_dtype)


def random_blob(o, D, F, rng, off, stride):
    gate = config0_matrix(o, F, D, rng)
    up = config0_matrix(o, F, D, rng)
    down = config0_matrix(o, D, F, rng)
    return o.pack_blob(gate, up, down, off, stride), (gate, up, down)


def quantized_blob(o, D, F, rng_uniform, off, stride):
    """Blob built the way the reference's tests build one: uniform weights through the quantiser
    (Tests/TurboFieldfare/Core/Kernels/MoE/MoEFusedFFNTests.swift:161-197)."""
    gate = o.quantize_rows(np.stack([rng_uniform(-0.5, 0.5, D) for _ in range(F)]), 4)
    up = o.quantize_rows(np.stack([rng_uniform(-0.5, 0.5, D) for _ in range(F)]), 4)
    down = o.quantize_rows(np.stack([rng_uniform(-0.5, 0.5, F) for _ in range(D)]), 4)
    return o.pack_blob(gate, up, down, off, stride), (gate, up, down)


def capi_offsets(off):
    from turbo_fieldfare_b200._capi import ExpertOffsets
    return ExpertOffsets(off.gate_w, off.gate_s, off.gate_b, off.up_w, off.up_s, off.up_b,
                         off.down_w, off.down_s, off.down_b)


def blob_table(blob_tensors):
    """Device table of blob base pointers (the argument buffer of Metal/MoE/moe.metal:74-76)."""
    import torch
    return torch.tensor([b.data_ptr() for b in blob_tensors], dtype=torch.int64, device="cuda")
