"""Host-side check of the error bound behind the two-launch prefill router (csrc/router_tensor.cuh).

A numpy model of router_approx_kernel (fp16 split of x * 2^10, exact products, k = 16 steps accumulated in fp32, the
per-group scale/bias epilogue, the magnitude) is compared with the oracle's canonical fp32 logits
(oracle/tf_oracle.c: tfo_router_logits, the order of Metal/MoE/moe.metal:135-185). The tensor-core adder is modelled
twice: rounding every step to nearest, and truncating every step toward zero (the pessimistic reading of an adder
that aligns and truncates its addends). In both models the distance from the canonical logit must stay well inside
eps = 2^-13 * magnitude + 2^-22 |v|, and the candidate rule built on eps must keep every canonical top-8 expert."""
import numpy as np
import pytest

from helpers import config0_matrix

REL_ERROR = 2.0 ** -13
PRESCALE = 1024.0
GROUP = 64


def _to_f32(x64, truncate):
    r = x64.astype(np.float32)
    if truncate:
        over = np.abs(r.astype(np.float64)) > np.abs(x64)
        r = np.where(over, np.nextafter(r, np.float32(0.0)), r).astype(np.float32)
    return r


def _approx_model(o, mat, h16, eff16, truncate):
    """(approximate logits, magnitudes) [T, E] in units of x, as router_approx_kernel writes them."""
    q = mat.packed.astype(np.float64)                                     # [E, D] codes 0...255, exact in fp16
    s = o.bf16_to_f32(mat.scales).astype(np.float64)                      # [E, G]
    b = o.bf16_to_f32(mat.biases).astype(np.float64)
    x = (o.f16_to_f32(h16) * o.bf16_to_f32(eff16)[None, :]).astype(np.float32)      # the canonical fp32 product
    y = (x * np.float32(PRESCALE)).astype(np.float32)
    hi = o.f16_to_f32(o.f32_to_f16(y))
    lo = o.f16_to_f32(o.f32_to_f16((y - hi).astype(np.float32)))
    T, D = y.shape
    E, G = s.shape
    acc = np.zeros((T, E), np.float32)
    mag = np.zeros((T, E), np.float64)
    for g in range(G):
        P = np.zeros((T, E), np.float32)
        for step in range(GROUP // 16):
            cols = slice(g * GROUP + step * 16, g * GROUP + step * 16 + 16)
            for part in (hi, lo):                                         # two MMAs per step, same accumulator
                block = part[:, cols].astype(np.float64) @ q[:, cols].T   # exact: 16 products of <= 2^8 * 2^11 bits
                P = _to_f32(P.astype(np.float64) + block, truncate)
        xs = y[:, g * GROUP:(g + 1) * GROUP].astype(np.float32).sum(axis=1, dtype=np.float32)
        xa = np.abs(y[:, g * GROUP:(g + 1) * GROUP]).astype(np.float32).sum(axis=1, dtype=np.float32) + np.float32(0.015625)
        inner = _to_f32(b[None, :, g] * xs[:, None].astype(np.float64) + acc.astype(np.float64), False)     # fma(b, xs, acc)
        acc = _to_f32(s[None, :, g] * P.astype(np.float64) + inner.astype(np.float64), False)               # fma(s, P, .)
        mag += (255.0 * np.abs(s[:, g]) + np.abs(b[:, g]))[None, :] * xa[:, None].astype(np.float64)
    return acc.astype(np.float64) / PRESCALE, mag / PRESCALE


def _cases(o, rng, E, D):
    mat = config0_matrix(o, E, D, rng, bits=8)
    yield "benchmark distributions", mat, rng.standard_normal((24, D)).astype(np.float32)
    # scales spread over three decades between groups, heavy-tailed activations
    wild = config0_matrix(o, E, D, rng, bits=8)
    sc = o.bf16_to_f32(wild.scales) * (10.0 ** rng.uniform(-1.5, 1.5, wild.scales.shape)).astype(np.float32)
    wild.scales[:] = o.f32_to_bf16(sc)
    wild.biases[:] = o.f32_to_bf16((-128.0 * o.bf16_to_f32(wild.scales)).astype(np.float32))
    yield "wild scales, heavy tails", wild, np.clip(rng.standard_cauchy((24, D)), -200, 200).astype(np.float32)
    # activations whose low half is subnormal in fp16 after the prescale, and rows that cancel almost completely
    yield "tiny activations", mat, (1e-4 * rng.standard_normal((24, D))).astype(np.float32)
    flat = config0_matrix(o, E, D, rng, bits=8)
    flat.packed[:] = 128                                                  # w = 128 s + b ~ 0: the two terms of a group cancel
    yield "cancelling groups", flat, rng.standard_normal((24, D)).astype(np.float32)


@pytest.mark.parametrize("truncate", [False, True])
def test_tensor_core_logits_stay_inside_the_bound(oracle, truncate):
    o = oracle
    rng = np.random.default_rng(4242)
    E, D, K = 64, 2816, 8
    eff = o.f32_to_bf16((rng.uniform(0.5, 1.5, D) / np.sqrt(D)).astype(np.float32))
    for name, mat, x in _cases(o, rng, E, D):
        h16 = o.f32_to_f16(x)
        canonical = o.router_logits(mat, h16, eff).astype(np.float64)
        approx, mag = _approx_model(o, mat, h16, eff, truncate)
        eps = REL_ERROR * mag + np.abs(approx) * 2.0 ** -22
        ratio = np.abs(approx - canonical) / eps
        assert np.all(np.isfinite(ratio)), name
        # eps is a worst-case bound (every rounding in the same direction); the modelled distances are 2e-5 to 2e-3 of it
        assert ratio.max() < 0.05, f"{name}: |approximate - canonical| reaches {ratio.max():.4f} eps"
        # the candidate rule: nothing outside the candidates may be in the canonical top k
        lower, upper = approx - eps, approx + eps
        lb = np.sort(lower, axis=1)[:, -K]
        cand = upper >= lb[:, None]
        top = np.argsort(-canonical, axis=1, kind="stable")[:, :K]
        assert np.all(np.take_along_axis(cand, top, axis=1)), name
        assert cand.sum(axis=1).min() >= K
