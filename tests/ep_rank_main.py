"""One rank of the 2-GPU expert-parallel check (launched by tests/test_gpu_ep.py with torchrun): every rank
runs its own tokens through the expert-parallel stack and through a private single-GPU stack with the
same seeds, and writes the relative L2 difference."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def main(out_dir: str) -> None:
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from turbo_fieldfare_b200.ep import ExpertParallelStack
    from turbo_fieldfare_b200.kernels import TurboContext
    from turbo_fieldfare_b200.stack import MoEStack
    ctx = TurboContext(local)
    dims = dict(layers=2, d=256, f=128, fs=192, num_experts=16, top_k=8, seed=5, align=256)
    ep_stack = ExpertParallelStack(ctx, **dims)
    ref_stack = MoEStack(ctx, **dims)
    worst = 0.0
    for T, fixed in ((6, True), (70, False)):
        g = torch.Generator().manual_seed(17 + rank + T)
        h = torch.randn(T, 256, generator=g).half().cuda()
        h_ep, h_ref = h.clone(), h.clone()
        ep_stack.forward(h_ep, T, ep_stack.buffers(T, fixed))
        ref_stack.forward(h_ref, T, ref_stack.workspace(T))
        torch.cuda.synchronize()
        a, b = h_ref.float(), h_ep.float()
        worst = max(worst, float((a - b).norm() / a.norm()))
    # decode-sized steps with the exchange over peer memory: eager, then the whole step as a replayed CUDA graph
    for T in (1, 6):
        g = torch.Generator().manual_seed(29 + rank + T)
        h = torch.randn(T, 256, generator=g).half().cuda()
        h_ref = h.clone()
        ref_stack.forward(h_ref, T, ref_stack.workspace(T))
        buf = ep_stack.buffers(T, True, peer=True)
        h_ep = h.clone()
        ep_stack.forward(h_ep, T, buf)
        torch.cuda.synchronize()
        a = h_ref.float()
        worst = max(worst, float((a - h_ep.float()).norm() / a.norm()))
        static_h = h.clone()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            ep_stack.forward(static_h, T, buf)
        for _ in range(2):
            static_h.copy_(h)
            graph.replay()
            torch.cuda.synchronize()
            worst = max(worst, float((a - static_h.float()).norm() / a.norm()))
        buf.close()
    # a prefill-sized block without the host in the layer loop: fixed-capacity slots over peer memory, and the owner's
    # expert phase on the tensor cores (most slots of the receive area are empty)
    ctx.set_ep_tensorcore_min_rows_per_expert(1)
    for T in (70, 300):
        g = torch.Generator().manual_seed(41 + rank + T)
        h = torch.randn(T, 256, generator=g).half().cuda()
        h_ref, h_ep = h.clone(), h.clone()
        ref_stack.forward(h_ref, T, ref_stack.workspace(T))
        buf = ep_stack.buffers(T, True, peer=True)
        ep_stack.forward(h_ep, T, buf)
        torch.cuda.synchronize()
        a = h_ref.float()
        worst = max(worst, float((a - h_ep.float()).norm() / a.norm()))
        buf.close()
    ctx.set_ep_tensorcore_min_rows_per_expert(0xFFFFFFFF)
    # experts placed by the load of a calibration batch: the shards level out, the load per original expert id and the
    # outputs stay those of the contiguous placement
    from turbo_fieldfare_b200.ep import balanced_placement, shard_imbalance
    g = torch.Generator().manual_seed(53 + rank)
    calib = torch.randn(96, 256, generator=g).half().cuda()
    exact = ep_stack.buffers(96, False)
    load = ep_stack.expert_load(calib, 96, exact)
    assert int(load.sum()) == 2 * 2 * 96 * 8
    placement = balanced_placement(ctx.lib, load, 2)
    assert np.all(shard_imbalance(load, placement, 2) <= shard_imbalance(load, None, 2) + 1e-12)
    ep_stack.set_placement(placement)
    assert np.array_equal(ep_stack.expert_load(calib, 96, exact), load)
    for T, fixed, peer in ((70, False, False), (6, True, True), (1, True, True)):
        g = torch.Generator().manual_seed(67 + rank + T)
        h = torch.randn(T, 256, generator=g).half().cuda()
        h_ref, h_ep = h.clone(), h.clone()
        ref_stack.forward(h_ref, T, ref_stack.workspace(T))
        buf = ep_stack.buffers(T, fixed, peer=peer)
        ep_stack.forward(h_ep, T, buf)
        torch.cuda.synchronize()
        a = h_ref.float()
        worst = max(worst, float((a - h_ep.float()).norm() / a.norm()))
        buf.close()
    assert ctx.device_status() == 0
    np.save(os.path.join(out_dir, f"err_{rank}.npy"), np.array(worst))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])
