"""Expert parallelism: experts sharded 128/N per GPU, tokens data-parallel, one dispatch and one combine exchange
per layer.

The reference is single-GPU (``Infrastructure/Metal/MetalContext.swift:51-71``); the multi-GPU form lives in the
library behind the C ABI (``tf_ep_create``, ``tf_ep_buffers_create``, ``tf_moe_block_forward_ep``,
``tf_stack_forward_ep``: communicator, exchange buffers, the per-layer loop and every collective). This module is the
thin Python caller: it builds the synthetic sharded weights, hands the NCCL unique id from rank 0 to the other ranks
over ``torch.distributed`` (any host channel would do) and forwards the calls. :func:`plan_dispatch` is the index
arithmetic of the pack kernel in numpy, used by the CPU tests.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch
import torch.distributed as dist

from . import _capi
from .kernels import TurboContext, _ptr, _stream
from .stack import (GEMMA4_D, GEMMA4_E, GEMMA4_F, GEMMA4_FS, GEMMA4_K, GEMMA4_LAYERS, BLOB_ALIGN, ExpertPool,
                    MoEBlockLayer, _bf16_bits)

EMPTY_SLOT = 0xFFFFFFFF


def plan_dispatch(indices: np.ndarray, experts_per_rank: int, n_ranks: int, capacity: int = 0):
    """Numpy statement of what ``tf_ep_pack`` computes for router output ``indices`` [T, K].

    Returns (send_token [slots], send_expert_local [slots], inverse_perm [T*K], send_counts [n_ranks]).
    Slots are ordered by (destination rank, expert, token, rank); with ``capacity`` > 0 the layout is
    [n_ranks][capacity] and unused slots carry ``EMPTY_SLOT``."""
    T, K = indices.shape
    flat = indices.reshape(-1).astype(np.int64)
    order = np.lexsort((np.tile(np.arange(K), T), np.repeat(np.arange(T), K), flat))   # (expert, token, rank)
    dst = flat[order] // experts_per_rank
    send_counts = np.bincount(dst, minlength=n_ranks).astype(np.int64)
    if capacity:
        if send_counts.max(initial=0) > capacity:
            raise ValueError(f"destination overflow: {send_counts.max()} rows > capacity {capacity}")
        slots = n_ranks * capacity
        base = np.concatenate([[0], np.cumsum(send_counts)[:-1]])
        slot_of = dst * capacity + (np.arange(order.size) - base[dst])
    else:
        slots = order.size
        slot_of = np.arange(order.size)
    send_token = np.full(slots, -1, dtype=np.int64)
    send_expert_local = np.full(slots, EMPTY_SLOT, dtype=np.uint32)
    send_token[slot_of] = order // K
    send_expert_local[slot_of] = (flat[order] % experts_per_rank).astype(np.uint32)
    inverse = np.empty(T * K, dtype=np.uint32)
    inverse[order] = slot_of.astype(np.uint32)
    return send_token, send_expert_local, inverse, send_counts


TF_EP_EXACT, TF_EP_FIXED_NCCL, TF_EP_FIXED_PEER = 0, 1, 2


def balanced_placement(lib, counts: np.ndarray, n_ranks: int) -> np.ndarray:
    """``tf_ep_balanced_placement``: per layer, the renumbering (new id -> original id) that spreads the measured
    load ``counts`` [layers, experts] evenly over ``n_ranks`` contiguous shards."""
    c = np.ascontiguousarray(counts, dtype=np.uint64)
    if c.ndim != 2:
        raise ValueError("counts must be [layers, experts]")
    out = np.zeros(c.shape, dtype=np.uint32)
    status = lib.tf_ep_balanced_placement(c.ctypes.data, c.shape[0], c.shape[1], n_ranks, out.ctypes.data)
    if status != 0:
        raise ValueError(f"tf_ep_balanced_placement: status {status} ({c.shape[1]} experts over {n_ranks} ranks)")
    return out


def shard_imbalance(counts: np.ndarray, placement: np.ndarray | None, n_ranks: int) -> np.ndarray:
    """Per layer: rows of the most loaded shard / rows of the average shard under ``placement`` (None: contiguous)."""
    c = np.asarray(counts, dtype=np.float64)
    if placement is not None:
        c = np.take_along_axis(c, np.asarray(placement, dtype=np.int64), axis=1)
    per_rank = c.reshape(c.shape[0], n_ranks, -1).sum(axis=2)
    return per_rank.max(axis=1) / np.maximum(per_rank.mean(axis=1), 1e-30)


class ExpertParallelStack:
    """Synthetic stack of MoE blocks with the routed experts sharded over the ranks of ``group``.

    Router, gains, shared expert and norm weights are replicated (seeded independently of the rank);
    expert blobs are seeded by their global id, so every world size computes with the same weights."""

    def __init__(self, context: TurboContext, layers: int = GEMMA4_LAYERS, d: int = GEMMA4_D, f: int = GEMMA4_F,
                 fs: int = GEMMA4_FS, num_experts: int = GEMMA4_E, top_k: int = GEMMA4_K, seed: int = 2026,
                 eps: float = 1e-6, align: int = BLOB_ALIGN, group=None):
        self.context = context
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if num_experts % self.world:
            raise ValueError(f"{num_experts} experts do not divide over {self.world} ranks")
        self.local_experts = num_experts // self.world
        self.dims = dict(layers=layers, d=d, f=f, fs=fs, num_experts=num_experts, top_k=top_k)
        self.eps = eps
        self.seed = seed
        self.placement = None                     # [layers, experts] new id -> original id (None: contiguous shards)
        self.pool = ExpertPool(context, layers, self.local_experts, d, f, align)
        self.pool.fill_synthetic(seed, global_experts=num_experts, expert_offset=self.rank * self.local_experts)
        rng = np.random.default_rng(seed)
        self.layers, self.norm_weights = [], []
        for l in range(layers):
            layer = MoEBlockLayer(context, self.pool, l, d, f, fs, num_experts, top_k)
            layer.fill_synthetic(seed * 1000 + l)
            self.layers.append(layer)
            w = (1.0 + 0.02 * rng.standard_normal(d)).astype(np.float32)
            self.norm_weights.append(torch.from_numpy(_bf16_bits(w).view(np.int16)).cuda())
        torch.cuda.synchronize()
        self._build()
        # the communicator: rank 0 makes the NCCL id, the host channel (torch.distributed here) carries it
        lib = context.lib
        uid = C.create_string_buffer(128)
        if self.world > 1:
            if self.rank == 0:
                context.check(lib.tf_ep_unique_id(uid))
            box = [bytes(uid.raw)]
            dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
            uid = C.create_string_buffer(box[0], 128)
        handle = C.c_void_p()
        context.check(lib.tf_ep_create(context.handle, uid, self.rank, self.world, C.byref(handle)))
        self.handle = handle

    def _build(self) -> None:
        n = len(self.layers)
        self._c_layers = (_capi.MoELayer * n)(*[l.c_struct() for l in self.layers])
        self._c_norms = (C.c_void_p * n)(*[w.data_ptr() for w in self.norm_weights])

    def set_logit_bias(self, bias) -> None:
        for l in self.layers:
            l.set_logit_bias(bias)
        self._build()

    def set_placement(self, placement: np.ndarray | None) -> None:
        """Place the experts by ``placement`` [layers, experts] (new id -> original id; rank r owns the new ids
        [r * E / world, (r + 1) * E / world)): the routers' rows are renumbered and this rank's pool is refilled with the
        experts it now owns. Every rank must pass the same table. Outputs do not change."""
        E, L = self.dims["num_experts"], self.dims["layers"]
        if placement is None:
            self.pool.fill_synthetic(self.seed, global_experts=E, expert_offset=self.rank * self.local_experts)
        else:
            placement = np.ascontiguousarray(placement, dtype=np.uint32)
            if placement.shape != (L, E):
                raise ValueError(f"placement must be [{L}, {E}], got {placement.shape}")
            mine = placement[:, self.rank * self.local_experts:(self.rank + 1) * self.local_experts]
            self.pool.fill_synthetic(self.seed, global_experts=E, original_ids=mine)
        for l, layer in enumerate(self.layers):
            layer.set_placement(None if placement is None else placement[l])
        self.placement = placement
        torch.cuda.synchronize()
        self._build()

    def expert_load(self, hidden: torch.Tensor, tokens: int, buf: "EPBuffers", stream=None) -> np.ndarray:
        """Routed pairs per (layer, ORIGINAL expert id) that ``hidden`` [tokens, d] produces, summed over the ranks'
        batches: the layer loop of ``forward`` run one layer at a time with the router's output read back after each
        (a calibration pass, not a fast path). Collective; ``buf`` must be exact-count buffers."""
        from .kernels import RMSNorm
        E, L, d = self.dims["num_experts"], self.dims["layers"], self.dims["d"]
        norm = RMSNorm(self.context)
        h = hidden[:tokens].clone()
        x, y = torch.empty_like(h), torch.empty_like(h)
        counts = np.zeros((L, E), dtype=np.int64)
        for l in range(L):
            norm.encode(h, self.norm_weights[l], x, tokens, d, eps=self.eps, stream=stream)
            self.block_forward(l, x, y, tokens, buf, stream)
            idx, _ = buf.routing(tokens)
            new_ids = np.bincount(idx.ravel().astype(np.int64), minlength=E)
            if self.placement is None:
                counts[l] = new_ids
            else:
                counts[l, self.placement[l].astype(np.int64)] = new_ids
            h += y
        if self.world > 1:
            t = torch.from_numpy(counts).cuda()
            dist.all_reduce(t, group=self.group)
            counts = t.cpu().numpy()
        return counts

    def buffers(self, max_tokens: int, fixed_capacity: bool, peer: bool = False) -> "EPBuffers":
        """``fixed_capacity``: static shapes and no host synchronisation (decode-sized batches); otherwise exact row
        counts with one read-back per layer (prefill). ``peer``: the fixed-capacity exchange runs over peer memory
        (plain kernels, capturable in a CUDA graph) instead of NCCL. Collective: every rank must ask for the same
        buffers in the same order."""
        mode = TF_EP_EXACT if not fixed_capacity else (TF_EP_FIXED_PEER if peer else TF_EP_FIXED_NCCL)
        return EPBuffers(self, max_tokens, mode)

    def forward(self, hidden: torch.Tensor, tokens: int, buf: "EPBuffers", stream=None) -> None:
        """hidden: fp16 [tokens, d] on the device, updated in place: x = rmsnorm(h) * w_l; h = h + block_l(x)."""
        ctx = self.context
        ctx.check(ctx.lib.tf_stack_forward_ep(self.handle, _stream(stream), self._c_layers, self._c_norms, len(self.layers),
                                              self.eps, _ptr(hidden), tokens, buf.handle))

    def block_forward(self, l: int, x: torch.Tensor, y: torch.Tensor, tokens: int, buf: "EPBuffers", stream=None) -> None:
        ctx = self.context
        ctx.check(ctx.lib.tf_moe_block_forward_ep(self.handle, _stream(stream), C.byref(self._c_layers[l]), _ptr(x), _ptr(y), tokens,
                                                  buf.handle))

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.context.lib.tf_ep_destroy(self.handle)
            self.handle = None
        self.pool.close()


class EPBuffers:
    """``tf_ep_buffers``: device buffers of one expert-parallel forward for up to ``max_tokens`` local tokens."""

    def __init__(self, stack: ExpertParallelStack, max_tokens: int, mode: int):
        dm = stack.dims
        self.stack, self.max_tokens = stack, max_tokens
        ctx = stack.context
        handle = C.c_void_p()
        ctx.check(ctx.lib.tf_ep_buffers_create(stack.handle, max_tokens, dm["d"], dm["f"], dm["fs"], dm["top_k"], dm["num_experts"],
                                               mode, C.byref(handle)))
        self.handle = handle
        self.mode = int(ctx.lib.tf_ep_buffers_mode(handle))
        self.fixed = self.mode != TF_EP_EXACT
        self.peer = self.mode == TF_EP_FIXED_PEER       # False after a collective fallback to NCCL

    def routing(self, tokens: int):
        """(indices uint32 [tokens, K], weights fp16 bits [tokens, K]) of the last forward's last layer, on the host."""
        from .stack import device_view_u8
        lib = self.stack.context.lib
        ws = lib.tf_ep_buffers_workspace(self.handle)
        k = self.stack.dims["top_k"]
        idx = device_view_u8(lib.tf_workspace_indices(ws), tokens * k * 4).cpu().numpy().view(np.uint32).reshape(tokens, k)
        w = device_view_u8(lib.tf_workspace_weights(ws), tokens * k * 2).cpu().numpy().view(np.uint16).reshape(tokens, k)
        return idx.copy(), w.copy()

    def close(self) -> None:
        """Frees the buffers (collective when peers are mapped: every rank must call it)."""
        if getattr(self, "handle", None):
            self.stack.context.lib.tf_ep_buffers_destroy(self.handle)
            self.handle = None
