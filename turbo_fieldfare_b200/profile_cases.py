"""Small, self-contained GPU cases for profiling one kernel at a time under ncu.

    python -m turbo_fieldfare_b200.profile_cases block --tokens 64 --layers 2 --iters 3
    python -m turbo_fieldfare_b200.profile_cases gemv --rows 262144 --iters 3
    python -m turbo_fieldfare_b200.profile_cases qmm --tokens 4096 --rows 4224 --iters 3

Each case holds well under a few GB on the device, streams more than the 126 MB L2 per
launch (one layer of experts is 430 MB), and launches only a handful of kernels, so that a
capture of one to three launches ends by itself.
"""
from __future__ import annotations

import argparse

import torch

from .kernels import DequantInt4GEMV, TurboContext
from .stack import AffineTensor, MoEStack


def case_block(args) -> None:
    ctx = TurboContext(0)
    if args.tensor_min > 0:
        ctx.set_tensorcore_min_tokens(args.tensor_min)
    stack = MoEStack(ctx, layers=args.layers, seed=3)
    ws = stack.workspace(args.tokens)
    h = torch.randn(args.tokens, 2816, device="cuda").half()
    if args.zipf > 0:
        import numpy as np
        p = 1.0 / (np.random.default_rng(0).permutation(128) + 1) ** args.zipf
        stack.set_logit_bias(np.log(p / p.sum()).astype(np.float32))
    for _ in range(args.warm):
        stack.forward(h, args.tokens, ws)
    times = []
    for _ in range(args.iters):
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        stack.forward(h, args.tokens, ws)
        t1.record()
        torch.cuda.synchronize()
        times.append(t0.elapsed_time(t1))
    print(f"block case done: tokens={args.tokens} layers={args.layers} iters={args.iters} launches={ctx.launch_count} "
          f"status={ctx.device_status()} ms_per_forward={[round(t, 3) for t in times]}")


def case_gemv(args) -> None:
    ctx = TurboContext(0)
    mat = AffineTensor(args.rows, 2816, 4)
    mat.fill_synthetic(ctx, 5)
    x = torch.randn(2816, device="cuda").half()
    y = torch.zeros(args.rows, dtype=torch.float16, device="cuda")
    k = DequantInt4GEMV(ctx)
    launch = lambda: k.encode(mat.buffer, mat.buffer, mat.buffer, x, y, args.rows, 2816, scales_offset=mat.s_off, biases_offset=mat.b_off)
    for _ in range(args.warm):
        launch()
    times = []
    for _ in range(args.iters):
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(10):
            launch()
        t1.record()
        torch.cuda.synchronize()
        times.append(t0.elapsed_time(t1) / 10)
    nbytes = mat.w_bytes + 2 * mat.sb_bytes
    print(f"gemv case done: rows={args.rows} bytes={nbytes} ms={[round(t, 4) for t in times]} GBps={nbytes / min(times) / 1e6:.0f}")


def case_lmhead(args) -> None:
    """Greedy LM head (final RMSNorm, tied int4 head of --rows x 2816, argmax): four launches per token."""
    from .kernels import LMHeadChainInt4
    ctx = TurboContext(0)
    mat = AffineTensor(args.rows, 2816, 4)
    mat.fill_synthetic(ctx, 5)
    hidden = torch.randn(2816, device="cuda").half()
    norm = torch.ones(2816, device="cuda").bfloat16()
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    op = LMHeadChainInt4(ctx)
    launch = lambda: op.encode_greedy_decode(hidden, norm, mat.buffer, mat.buffer, mat.buffer, out, 2816, args.rows,
                                             scales_offset=mat.s_off, biases_offset=mat.b_off)
    for _ in range(max(args.warm, 1)):
        launch()
    times = []
    for _ in range(args.iters):
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(10):
            launch()
        t1.record()
        torch.cuda.synchronize()
        times.append(t0.elapsed_time(t1) / 10)
    nbytes = mat.w_bytes + 2 * mat.sb_bytes
    print(f"lmhead case done: rows={args.rows} bytes={nbytes} token={int(out.item())} status={ctx.device_status()} "
          f"ms={[round(t, 4) for t in times]} GBps={nbytes / min(times) / 1e6:.0f}")


def case_qmm(args) -> None:
    """Dense int4 QMM on the tensor cores: --tokens rows of activations against a [--rows, 2816] weight matrix."""
    from .kernels import MPPPrefillInt4QMM
    ctx = TurboContext(0)
    k = args.cols
    mat = AffineTensor(args.rows, k, 4)
    mat.fill_synthetic(ctx, 5)
    x = torch.randn(args.tokens, k, device="cuda").half()
    y = torch.zeros(args.tokens, args.rows, dtype=torch.float16, device="cuda")
    op = MPPPrefillInt4QMM(ctx)
    launch = lambda: op.encode(mat.buffer, mat.buffer, mat.buffer, x, y, args.tokens, args.rows, k,
                               scales_offset=mat.s_off, biases_offset=mat.b_off)
    for _ in range(args.warm):            # clocks ramp up only under sustained load
        launch()
    times = []
    for _ in range(args.iters):           # each sample: 20 launches back to back, so the host's launch cost hides behind the GPU
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(20):
            launch()
        t1.record()
        torch.cuda.synchronize()
        times.append(t0.elapsed_time(t1) / 20)
    nbytes = mat.w_bytes + 2 * mat.sb_bytes
    best = min(times)
    print(f"qmm case done: tokens={args.tokens} rows={args.rows} cols={k} weight_bytes={nbytes} status={ctx.device_status()} "
          f"ms={[round(t, 4) for t in times]} weight_GBps={nbytes / best / 1e6:.0f} TFLOPs={2 * args.tokens * args.rows * k / best / 1e9:.0f}")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["block", "gemv", "qmm", "lmhead"])
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--rows", type=int, default=262144)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--cols", type=int, default=2816)
    ap.add_argument("--warm", type=int, default=0, help="untimed launches before the timed ones")
    ap.add_argument("--tensor-min", type=int, default=0, help="block case: smallest token count that takes the tensor-core path")
    ap.add_argument("--zipf", type=float, default=0.0, help="router logit bias log(p), p ~ 1/rank^zipf (0 = none)")
    args = ap.parse_args()
    {"block": case_block, "gemv": case_gemv, "qmm": case_qmm, "lmhead": case_lmhead}[args.case](args)


if __name__ == "__main__":
    main()
