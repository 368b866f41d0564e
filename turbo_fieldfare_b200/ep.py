"""Expert parallelism: experts sharded 128/N per GPU, tokens data-parallel, one dispatch and one combine
all-to-all per layer over NCCL (``torch.distributed``).

The reference is single-GPU (``Infrastructure/Metal/MetalContext.swift:51-71``); this module is the
multi-GPU form the build adds. Per layer:

    tf_ep_dispatch   router, top-8, device grouping over the global experts, pack rows by owner rank
    all-to-all       expert ids and activation rows to the owners
    tf_ep_experts    owners group the received rows by local expert and run gate/up/GeGLU/down
    all-to-all       result rows back to the tokens' home ranks
    tf_ep_finish     shared expert (replicated weights) + weighted combine in rank order

Two exchange layouts: a fixed capacity per destination (static shapes, no host synchronisation; used for
decode-sized batches) and exact split sizes read back from the device (one synchronisation per layer;
used for prefill). :func:`plan_dispatch` is the same index arithmetic in numpy, used by the CPU tests.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch
import torch.distributed as dist

from . import _capi
from .kernels import DeviceRoutes, TurboContext, _ptr, _stream
from .stack import (GEMMA4_D, GEMMA4_E, GEMMA4_F, GEMMA4_FS, GEMMA4_K, GEMMA4_LAYERS, BLOB_ALIGN, ExpertPool,
                    MoEBlockLayer, Workspace, _bf16_bits)

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
        # exact-split exchanges of at least this many rows run their experts on the tensor cores (256 tokens x top-8)
        self.tensorcore_min_rows = 2048
        self.dims = dict(layers=layers, d=d, f=f, fs=fs, num_experts=num_experts, top_k=top_k)
        self.eps = eps
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
        self._c_layers = [l.c_struct() for l in self.layers]
        torch.cuda.synchronize()

    def set_logit_bias(self, bias) -> None:
        for l in self.layers:
            l.set_logit_bias(bias)
        self._c_layers = [l.c_struct() for l in self.layers]

    def buffers(self, max_tokens: int, fixed_capacity: bool, peer: bool = False) -> "EPBuffers":
        """``peer``: fixed-capacity buffers whose exchange runs over peer memory (plain kernels, capturable in a CUDA
        graph) instead of NCCL all-to-all calls. Collective: every rank must ask for the same buffers in the same order."""
        return EPBuffers(self, max_tokens, fixed_capacity, peer)

    def forward(self, hidden: torch.Tensor, tokens: int, buf: "EPBuffers", stream=None) -> None:
        """hidden: fp16 [tokens, d] on the device, updated in place: x = rmsnorm(h) * w_l; h = h + block_l(x)."""
        ctx, lib, d = self.context, self.context.lib, self.dims["d"]
        st = _stream(stream)
        y_prev = None
        for l, layer in enumerate(self._c_layers):
            ctx.check(lib.tf_residual_rmsnorm(ctx.handle, st, _ptr(hidden), _ptr(y_prev), _ptr(self.norm_weights[l]),
                                              _ptr(buf.x_norm), tokens, d, self.eps))
            self.block_forward(l, buf.x_norm, buf.y_block, tokens, buf, stream)
            y_prev = buf.y_block
        ctx.check(lib.tf_residual_rmsnorm(ctx.handle, st, _ptr(hidden), _ptr(y_prev), None, None, tokens, d, self.eps))

    def block_forward(self, l: int, x: torch.Tensor, y: torch.Tensor, tokens: int, buf: "EPBuffers", stream=None) -> None:
        ctx, lib = self.context, self.context.lib
        dm = self.dims
        d, f, K = dm["d"], dm["f"], dm["top_k"]
        st = _stream(stream)
        layer = self._c_layers[l]
        n_pairs = tokens * K
        cap = buf.capacity if buf.fixed else 0
        # fixed-capacity rows are D + 8 elements wide: the tail carries the expert id, one exchange moves both
        row_stride = buf.row_stride
        ctx.check(lib.tf_ep_dispatch(ctx.handle, st, C.byref(layer), _ptr(x), tokens, buf.ws.handle, self.local_experts,
                                     cap, _ptr(buf.send_rows), _ptr(buf.send_ids), _ptr(buf.inverse), row_stride))
        if buf.fixed and buf.peer:
            # rows (with their id tails) straight into the owners' receive areas; the launch ends with the flag barrier
            slots = recv_slots = self.world * cap
            ctx.check(lib.tf_ep_peer_push(ctx.handle, st, _ptr(buf.send_rows), row_stride, _ptr(buf.peer_bases), 0, row_stride,
                                          row_stride, None, d, self.world, self.rank, cap, buf.flags_offset, _ptr(buf.epoch)))
            recv_ids, recv_rows = buf.recv_ids, buf.recv_rows
        elif buf.fixed:
            slots = self.world * cap
            recv_slots = slots
            if self.world > 1:
                dist.all_to_all_single(buf.recv_rows[:slots * row_stride], buf.send_rows[:slots * row_stride], group=self.group)
                recv_ids, recv_rows = buf.recv_ids, buf.recv_rows
            else:
                recv_ids, recv_rows = buf.recv_ids, buf.send_rows
        else:
            # exact split sizes: one read-back of the per-expert counts per layer
            counts = buf.ws_counts(self.dims["num_experts"]).reshape(self.world, self.local_experts).sum(axis=1)
            send_splits = [int(c) for c in counts]
            if self.world > 1:
                sc = torch.tensor(send_splits, dtype=torch.int64, device="cuda")
                rc = torch.empty_like(sc)
                dist.all_to_all_single(rc, sc, group=self.group)
                recv_splits = [int(v) for v in rc.cpu()]
                recv_slots = sum(recv_splits)
                buf.ensure_recv(recv_slots)
                dist.all_to_all_single(buf.recv_ids[:recv_slots], buf.send_ids[:n_pairs], recv_splits, send_splits, group=self.group)
                dist.all_to_all_single(buf.recv_rows[:recv_slots * d].view(-1, d), buf.send_rows[:n_pairs * d].view(-1, d),
                                       recv_splits, send_splits, group=self.group)
                recv_ids, recv_rows = buf.recv_ids, buf.recv_rows
            else:
                recv_slots, recv_splits = n_pairs, send_splits
                recv_ids, recv_rows = buf.send_ids, buf.send_rows
                buf.ensure_recv(recv_slots)
        if not buf.fixed and recv_slots >= self.tensorcore_min_rows and d % 64 == 0 and f % 64 == 0:
            # prefill-sized exchange: every received slot holds a row, the experts run as tcgen05 grouped GEMMs
            buf.ensure_sorted(recv_slots)
            ctx.check(lib.tf_ep_experts_tensorcore(
                ctx.handle, st, self.pool.ptr(l, 0), self.pool.stride, C.byref(self.pool.offsets), _ptr(recv_rows),
                _ptr(recv_ids), recv_slots, self.local_experts, C.byref(buf.recv_routes.c_struct), _ptr(buf.zero_weights),
                _ptr(buf.one_weights), _ptr(buf.x_sorted), _ptr(buf.row_ids), _ptr(buf.inverse_sorted), _ptr(buf.acts),
                _ptr(buf.out_sorted), _ptr(buf.out_rows), d, f))
        else:
            ctx.check(lib.tf_ep_experts(ctx.handle, st, self.pool.ptr(l, 0), self.pool.stride, C.byref(self.pool.offsets),
                                        _ptr(recv_rows), _ptr(recv_ids), recv_slots, self.local_experts,
                                        C.byref(buf.recv_routes.c_struct), _ptr(buf.zero_weights), _ptr(buf.acts),
                                        _ptr(buf.out_rows), d, f, row_stride))
        if buf.fixed and buf.peer:
            # results back into the home ranks' areas (only the slots that held a row), and the second barrier
            ctx.check(lib.tf_ep_peer_push(ctx.handle, st, _ptr(buf.out_rows), d, _ptr(buf.peer_bases), buf.back_offset, d, d,
                                          _ptr(buf.recv_ids), 0, self.world, self.rank, cap, buf.flags_offset, _ptr(buf.epoch)))
            back = buf.back_rows
        elif self.world > 1:
            if buf.fixed:
                dist.all_to_all_single(buf.back_rows[:recv_slots * d], buf.out_rows[:recv_slots * d], group=self.group)
            else:
                dist.all_to_all_single(buf.back_rows[:n_pairs * d].view(-1, d), buf.out_rows[:recv_slots * d].view(-1, d),
                                       send_splits, recv_splits, group=self.group)
            back = buf.back_rows
        else:
            back = buf.out_rows
        ctx.check(lib.tf_ep_finish(ctx.handle, st, C.byref(layer), _ptr(x), tokens, buf.ws.handle, _ptr(back),
                                   _ptr(buf.inverse), _ptr(y)))

    def close(self) -> None:
        self.pool.close()


class EPBuffers:
    """Device buffers of one expert-parallel forward for up to ``max_tokens`` local tokens."""

    def __init__(self, stack: ExpertParallelStack, max_tokens: int, fixed_capacity: bool, peer: bool = False):
        dm = stack.dims
        self.peer = bool(peer and fixed_capacity)
        self._peer_handle, self._imported = None, []
        d, f, K, E = dm["d"], dm["f"], dm["top_k"], dm["num_experts"]
        self.stack, self.fixed, self.max_tokens = stack, fixed_capacity, max_tokens
        self.ws = Workspace(stack.context, max_tokens, d, f, dm["fs"], K, E)
        n_pairs = max_tokens * K
        self.capacity = n_pairs                     # a destination can receive every pair of this rank
        send_slots = stack.world * self.capacity if fixed_capacity else n_pairs
        i16 = dict(dtype=torch.float16, device="cuda")        # NCCL has no 16-bit integer type; the rows are fp16
        i32 = dict(dtype=torch.int32, device="cuda")
        self.row_stride = d + 8 if fixed_capacity else d        # fixed-capacity rows carry their expert id in the tail
        self.send_rows = torch.zeros(send_slots * self.row_stride, **i16)
        self.send_ids = torch.zeros(send_slots, **i32)
        self.inverse = torch.zeros(n_pairs, **i32)
        self.back_rows = torch.zeros(send_slots * d, **i16)
        self.x_norm = torch.zeros(max_tokens * d, **i16)
        self.y_block = torch.zeros(max_tokens * d, **i16)
        self.d, self.f = d, f
        self._recv_cap = 0
        self.ensure_recv(send_slots if fixed_capacity else max(n_pairs, 1))
        if self.peer:
            # Mapping is collective. If it fails on any rank (no peer access between two GPUs, IPC refused), every
            # rank drops back to the NCCL exchange together, so the ranks never disagree about the path.
            ok, why = 1, ""
            try:
                self._map_peer_buffers(send_slots)
            except Exception as exc:          # noqa: BLE001 - any failure means "no peer path on this machine"
                ok, why = 0, str(exc)
            if stack.world > 1:
                flag = torch.tensor([ok], dtype=torch.int32, device="cuda")
                dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=stack.group)
                ok_all = int(flag.item())
            else:
                ok_all = ok
            if not ok_all:
                self._drop_peer_buffers()
                self.peer = False
                self.peer_failure = why or "another rank could not map the peer buffers"
                self.ensure_recv_reset(send_slots)

    def _map_peer_buffers(self, slots: int) -> None:
        """One exchange buffer per rank: [receive area | return area | flags], mapped by every other rank (CUDA IPC).
        The receive and return areas replace ``recv_rows`` and ``back_rows``."""
        import ctypes as C
        from .stack import device_view_u8
        stack = self.stack
        ctx, lib = stack.context, stack.context.lib
        recv_bytes = slots * self.row_stride * 2
        back_bytes = slots * self.d * 2
        self.back_offset = (recv_bytes + 255) // 256 * 256
        self.flags_offset = (self.back_offset + back_bytes + 255) // 256 * 256
        total = self.flags_offset + 256
        handle = C.c_void_p()
        exported = C.create_string_buffer(64)
        status = lib.tf_peer_buffer_create(ctx.handle, total, C.byref(handle))
        if status == 0:
            self._peer_handle = handle
            status = lib.tf_peer_buffer_export(handle, exported)
        own = lib.tf_peer_buffer_ptr(handle) if status == 0 else 0
        bases = [own]
        if stack.world > 1:
            # every rank takes part in the gather even if its own allocation failed (None), so nobody waits alone
            gathered = [None] * stack.world
            dist.all_gather_object(gathered, bytes(exported.raw) if status == 0 else None, group=stack.group)
            if any(raw is None for raw in gathered):
                raise RuntimeError("a rank could not allocate or export its exchange buffer")
            bases = []
            for r, raw in enumerate(gathered):
                if r == stack.rank:
                    bases.append(own)
                    continue
                p = C.c_void_p()
                ctx.check(lib.tf_peer_buffer_import(ctx.handle, C.create_string_buffer(raw, 64), C.byref(p)))
                self._imported.append(p.value)
                bases.append(p.value)
        elif status != 0:
            ctx.check(status)
        self.peer_bases = torch.tensor(bases, dtype=torch.int64, device="cuda")
        self.epoch = torch.zeros(2, dtype=torch.int32, device="cuda")       # epoch counter, ticket of the push kernel
        self.recv_rows = device_view_u8(own, recv_bytes).view(torch.float16)
        self.back_rows = device_view_u8(own + self.back_offset, back_bytes).view(torch.float16)
        torch.cuda.synchronize()

    def _drop_peer_buffers(self) -> None:
        """Collective tear-down in the order CUDA IPC asks for: every rank closes its imports, all ranks meet, and only
        then does each rank free the buffer it exported (freeing exported memory that a peer still maps is undefined)."""
        ctx, lib = self.stack.context, self.stack.context.lib
        for p in self._imported:
            lib.tf_peer_buffer_release(ctx.handle, p)
        self._imported = []
        if self.stack.world > 1:
            dist.barrier(group=self.stack.group)
        if self._peer_handle is not None:
            lib.tf_peer_buffer_destroy(self._peer_handle)
            self._peer_handle = None

    def ensure_recv_reset(self, slots: int) -> None:
        """Receive and return buffers of the NCCL exchange (after a peer mapping that did not come up)."""
        self._recv_cap = 0
        self.ensure_recv(slots)
        self.back_rows = torch.zeros(slots * self.d, dtype=torch.float16, device="cuda")

    def close(self) -> None:
        """Unmaps the peers' buffers and frees this rank's (collective when peers are mapped)."""
        if not self.peer:
            return
        self.peer = False
        torch.cuda.synchronize()
        if self.stack.world > 1:
            dist.barrier(group=self.stack.group)     # nobody is still writing into a buffer that is about to go
        self._drop_peer_buffers()

    def ensure_recv(self, slots: int) -> None:
        if slots <= self._recv_cap:
            return
        cap = max(slots, int(self._recv_cap * 1.5))
        i16 = dict(dtype=torch.float16, device="cuda")
        i32 = dict(dtype=torch.int32, device="cuda")
        self.recv_rows = torch.zeros(cap * self.row_stride, **i16)
        self.recv_ids = torch.zeros(cap, **i32)
        self.out_rows = torch.zeros(cap * self.d, **i16)
        self.acts = torch.zeros(cap * self.f, **i16)
        self.zero_weights = torch.zeros(cap, **i16)
        self.recv_routes = DeviceRoutes(cap, 1, self.stack.local_experts)
        self._recv_cap = cap

    def ensure_sorted(self, slots: int) -> None:
        """Scratch of the tensor-core expert phase: expert-sorted rows in and out, the permutation, unit weights."""
        if slots <= getattr(self, "_sorted_cap", 0):
            return
        cap = max(slots, self._recv_cap)
        i16 = dict(dtype=torch.float16, device="cuda")
        i32 = dict(dtype=torch.int32, device="cuda")
        self.x_sorted = torch.zeros(cap * self.d, **i16)
        self.out_sorted = torch.zeros(cap * self.d, **i16)
        self.row_ids = torch.zeros(cap, **i32)
        self.inverse_sorted = torch.zeros(cap, **i32)
        self.one_weights = torch.ones(cap, **i16)
        self._sorted_cap = cap

    def ws_counts(self, num_experts: int) -> np.ndarray:
        """Per-expert pair counts of the last dispatch, read back from the device (synchronises)."""
        from .stack import device_view_u8
        lib = self.stack.context.lib
        routes = lib.tf_workspace_routes(self.ws.handle).contents
        return device_view_u8(routes.per_expert_counts, num_experts * 4).cpu().numpy().view(np.uint32).astype(np.int64)
