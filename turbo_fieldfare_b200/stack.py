"""HBM-resident expert pool, MoE block and layer stack over the C ABI.

Host-side mirror of what the reference spreads over ``Model`` (expert I/O,
``Runtime/Inference/ModelExpertIO.swift:21-142``), ``PreadExpertStreamer`` and the MoE
section of ``RealForwardRunner`` (``Runtime/Inference/RealForwardRunner.swift:902-1186,
1449-1693``). All experts live in GPU memory, so there is no cache plan, no
``pread`` and no CPU read-back of router ids.
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import torch

from . import _capi
from ._capi import ExpertOffsets, MoELayer, Projection
from .kernels import TurboContext, TFError, _ptr, _stream

GEMMA4_D, GEMMA4_F, GEMMA4_FS, GEMMA4_E, GEMMA4_K, GEMMA4_LAYERS = 2816, 704, 2112, 128, 8, 30
BLOB_ALIGN = 16384   # GTurboFormatV1 alignment (Sources/TurboFieldfareFormat/GTurboFormatV1.swift:3-22)


def expert_blob_layout(d: int, f: int, align: int = BLOB_ALIGN):
    """Offsets gate{W,S,B} | up{W,S,B} | down{W,S,B}, payload bytes and aligned stride
    (Sources/TurboFieldfareRepack/Core/Planning/RepackPlanner.swift:337-399)."""
    gw, gs = f * d // 2, f * (d // 64) * 2
    dw, ds = d * f // 2, d * (f // 64) * 2
    sizes = [gw, gs, gs, gw, gs, gs, dw, ds, ds]
    offs, cur = [], 0
    for s in sizes:
        offs.append(cur)
        cur += s
    stride = (cur + align - 1) // align * align
    return ExpertOffsets(*offs), cur, stride


class _RawDeviceBytes:
    """Exposes a raw device range through ``__cuda_array_interface__`` so torch can view it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False),
                                         "version": 2, "strides": None}


def device_view_u8(ptr: int, nbytes: int) -> torch.Tensor:
    """A uint8 tensor aliasing [ptr, ptr + nbytes) on the current device (no copy, no ownership)."""
    return torch.as_tensor(_RawDeviceBytes(ptr, nbytes), device="cuda")


class ExpertPool:
    """``tf_pool``: layers x experts blobs resident in HBM."""

    def __init__(self, context: TurboContext, layers: int, experts: int, d: int, f: int, align: int = BLOB_ALIGN):
        self.context, self.layers, self.experts, self.d, self.f = context, layers, experts, d, f
        self.offsets, self.payload, self.stride = expert_blob_layout(d, f, align)
        handle = C.c_void_p()
        context.check(context.lib.tf_expert_pool_create(context.handle, layers, experts, self.stride,
                                                        C.byref(self.offsets), C.byref(handle)))
        self.handle = handle

    def ptr(self, layer: int, expert: int = 0) -> int:
        p = self.context.lib.tf_expert_pool_ptr(self.handle, layer, expert)
        if not p:
            raise TFError(1, f"expert ({layer}, {expert}) out of range")
        return p

    @property
    def nbytes(self) -> int:
        return int(self.context.lib.tf_expert_pool_bytes(self.handle))

    def upload(self, layer: int, expert: int, blob: np.ndarray, stream=None) -> None:
        blob = np.ascontiguousarray(blob, dtype=np.uint8)
        self.context.check(self.context.lib.tf_expert_pool_upload(self.handle, _stream(stream), layer, expert,
                                                                  blob.ctypes.data, blob.size))
        torch.cuda.current_stream().synchronize()    # the host array may be freed by the caller

    def fill_synthetic(self, seed: int, stream=None, global_experts: int = 0, expert_offset: int = 0,
                       original_ids: np.ndarray | None = None) -> None:
        """Seeded synthetic blobs; a shard passes the global expert count and its first expert id so that
        it holds the same bytes as the corresponding slice of the unsharded pool. ``original_ids`` [layers, experts]
        instead names the expert of the unsharded pool that each slot holds (experts placed by load)."""
        lib, ctx = self.context.lib, self.context
        if original_ids is None:
            ctx.check(lib.tf_expert_pool_fill_synthetic(self.handle, _stream(stream), seed, self.d, self.f, global_experts,
                                                        expert_offset))
            return
        ids = np.ascontiguousarray(original_ids, dtype=np.uint32)
        if ids.shape != (self.layers, self.experts):
            raise ValueError(f"original_ids must be [{self.layers}, {self.experts}], got {ids.shape}")
        ctx.check(lib.tf_expert_pool_fill_synthetic_placed(self.handle, _stream(stream), seed, self.d, self.f,
                                                           global_experts or self.experts, ids.ctypes.data))

    def download(self, layer: int, expert: int) -> np.ndarray:
        """Copy one blob back to the host (tests use this to feed the oracle the exact bytes)."""
        return device_view_u8(self.ptr(layer, expert), self.stride).cpu().numpy()

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.context.lib.tf_expert_pool_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class AffineTensor:
    """A quantised matrix on the device: packed codes, scales, biases in one buffer."""

    def __init__(self, rows: int, cols: int, bits: int):
        self.rows, self.cols, self.bits = rows, cols, bits
        self.w_bytes = rows * cols // 2 if bits == 4 else rows * cols
        self.sb_bytes = rows * (cols // 64) * 2
        up = lambda v: (v + 255) // 256 * 256
        self.s_off = up(self.w_bytes)
        self.b_off = self.s_off + up(self.sb_bytes)
        self.buffer = torch.zeros(self.b_off + up(self.sb_bytes), dtype=torch.uint8, device="cuda")

    def projection(self) -> Projection:
        p = self.buffer.data_ptr()
        return Projection(p, 0, p, self.s_off, p, self.b_off, self.rows, self.cols)

    def fill_synthetic(self, context: TurboContext, seed: int, stream=None) -> None:
        p = self.buffer.data_ptr()
        context.check(context.lib.tf_fill_affine_synthetic(context.handle, _stream(stream), p, p + self.s_off,
                                                           p + self.b_off, self.rows, self.cols, self.bits, seed))

    def upload(self, packed: np.ndarray, scales: np.ndarray, biases: np.ndarray) -> None:
        host = np.zeros(self.buffer.numel(), dtype=np.uint8)
        host[:self.w_bytes] = np.ascontiguousarray(packed).view(np.uint8).reshape(-1)
        host[self.s_off:self.s_off + self.sb_bytes] = np.ascontiguousarray(scales).view(np.uint8).reshape(-1)
        host[self.b_off:self.b_off + self.sb_bytes] = np.ascontiguousarray(biases).view(np.uint8).reshape(-1)
        self.buffer.copy_(torch.from_numpy(host))

    def download(self):
        """(packed uint8 [rows, row_bytes], scales uint16 [rows, cols/64], biases uint16 [...])."""
        host = self.buffer.cpu().numpy()
        g = self.cols // 64
        packed = host[:self.w_bytes].reshape(self.rows, -1).copy()
        scales = host[self.s_off:self.s_off + self.sb_bytes].view(np.uint16).reshape(self.rows, g).copy()
        biases = host[self.b_off:self.b_off + self.sb_bytes].view(np.uint16).reshape(self.rows, g).copy()
        return packed, scales, biases


def _bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even bf16 bit patterns of a float32 array."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


class MoEBlockLayer:
    """Weights of one MoE block: router, gains, shared expert and a slice of the expert pool."""

    def __init__(self, context: TurboContext, pool: ExpertPool, layer_index: int, d: int, f: int, fs: int,
                 num_experts: int, top_k: int, shared_bits: int = 4):
        self.context, self.pool, self.layer_index = context, pool, layer_index
        self.d, self.f, self.fs, self.num_experts, self.top_k, self.shared_bits = d, f, fs, num_experts, top_k, shared_bits
        self.router = AffineTensor(num_experts, d, 8)
        self.shared_gate = AffineTensor(fs, d, shared_bits)
        self.shared_up = AffineTensor(fs, d, shared_bits)
        self.shared_down = AffineTensor(d, fs, shared_bits)
        eff = np.full(d, 1.0 / math.sqrt(d), dtype=np.float32)
        self.effective_scale = torch.from_numpy(_bf16_bits(eff).view(np.int16)).cuda()
        self.per_expert_scale = torch.from_numpy(_bf16_bits(np.ones(num_experts, np.float32)).view(np.int16)).cuda()
        self.logit_bias = None
        self.placement = None                     # new expert id -> original id (None: identity)
        self._router_original = None
        self._bias_original = None

    def fill_synthetic(self, seed: int) -> None:
        ctx = self.context
        self._router_original, self.placement = None, None
        self.router.fill_synthetic(ctx, seed * 16 + 1)
        self.shared_gate.fill_synthetic(ctx, seed * 16 + 2)
        self.shared_up.fill_synthetic(ctx, seed * 16 + 3)
        self.shared_down.fill_synthetic(ctx, seed * 16 + 4)

    def set_logit_bias(self, bias: np.ndarray | None) -> None:
        """``bias`` is indexed by the ORIGINAL expert id; it is stored in the placement's order."""
        self._bias_original = None if bias is None else np.ascontiguousarray(bias, np.float32)
        if bias is None:
            self.logit_bias = None
        else:
            order = self.placement if self.placement is not None else np.arange(self.num_experts)
            self.logit_bias = torch.from_numpy(self._bias_original[order].copy()).cuda()

    def set_placement(self, new_to_original: np.ndarray | None) -> None:
        """Renumber the experts: the router's row ``n`` becomes the row of expert ``new_to_original[n]`` (codes, scales,
        biases, per-expert scale, logit bias). The pool must store its slots in the same order. ``None`` restores the
        original numbering."""
        if self._router_original is None:
            self._router_original = self.router.download()
            self._pes_original = self.per_expert_scale.cpu().numpy().copy()
        if new_to_original is None:
            order = np.arange(self.num_experts)
            self.placement = None
        else:
            order = np.ascontiguousarray(new_to_original, dtype=np.int64)
            if sorted(order.tolist()) != list(range(self.num_experts)):
                raise ValueError("placement must be a permutation of the expert ids")
            self.placement = order
        packed, scales, biases = self._router_original
        self.router.upload(packed[order], scales[order], biases[order])
        self.per_expert_scale.copy_(torch.from_numpy(self._pes_original[order].copy()))
        if getattr(self, "_bias_original", None) is not None:
            self.logit_bias = torch.from_numpy(self._bias_original[order].copy()).cuda()

    def c_struct(self) -> MoELayer:
        return MoELayer(self.router.projection(), _ptr(self.effective_scale), _ptr(self.per_expert_scale),
                        _ptr(self.logit_bias), self.pool.ptr(self.layer_index, 0), self.pool.stride, self.pool.offsets,
                        self.shared_gate.projection(), self.shared_up.projection(), self.shared_down.projection(),
                        self.num_experts, self.d, self.f, self.fs, self.top_k, self.shared_bits)


class Workspace:
    """``tf_workspace``: device scratch for up to ``max_tokens`` tokens."""

    def __init__(self, context: TurboContext, max_tokens: int, d: int, f: int, fs: int, top_k: int, num_experts: int):
        self.context, self.max_tokens, self.top_k = context, max_tokens, top_k
        handle = C.c_void_p()
        context.check(context.lib.tf_workspace_create(context.handle, max_tokens, d, f, fs, top_k, num_experts,
                                                      C.byref(handle)))
        self.handle = handle

    def routing(self, tokens: int):
        """(indices uint32 [tokens, K], weights fp16 bits [tokens, K]) of the last forward, on the host."""
        lib = self.context.lib
        n = tokens * self.top_k
        idx = device_view_u8(lib.tf_workspace_indices(self.handle), n * 4).cpu().numpy()
        w = device_view_u8(lib.tf_workspace_weights(self.handle), n * 2).cpu().numpy()
        return (idx.view(np.uint32).reshape(tokens, self.top_k).copy(),
                w.view(np.uint16).reshape(tokens, self.top_k).copy())

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.context.lib.tf_workspace_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class MoEBlock:
    """One fused MoE block: ``y = shared(x) + sum_r w_r * routed_r(x)``."""

    def __init__(self, context: TurboContext, layer: MoEBlockLayer):
        self.context, self.layer = context, layer
        self._c = layer.c_struct()

    def refresh(self) -> None:
        self._c = self.layer.c_struct()

    def forward(self, x: torch.Tensor, y: torch.Tensor, tokens: int, ws: Workspace, stream=None) -> None:
        ctx = self.context
        ctx.check(ctx.lib.tf_moe_block_forward(ctx.handle, _stream(stream), C.byref(self._c), _ptr(x), self.layer.d,
                                               _ptr(y), self.layer.d, tokens, ws.handle))

    def forward_bf16(self, x: torch.Tensor, y: torch.Tensor, tokens: int, ws: Workspace, stream=None) -> None:
        """The same block on bf16 rows in and out (exact conversion to fp16 on entry, rounding to bf16 on exit)."""
        ctx = self.context
        ctx.check(ctx.lib.tf_moe_block_forward_bf16(ctx.handle, _stream(stream), C.byref(self._c), _ptr(x), self.layer.d,
                                                    _ptr(y), self.layer.d, tokens, ws.handle))


class MoEStack:
    """Synthetic stack of MoE blocks with RMSNorm between layers (attention omitted)."""

    def __init__(self, context: TurboContext, layers: int = GEMMA4_LAYERS, d: int = GEMMA4_D, f: int = GEMMA4_F,
                 fs: int = GEMMA4_FS, num_experts: int = GEMMA4_E, top_k: int = GEMMA4_K, seed: int = 2026,
                 eps: float = 1e-6, align: int = BLOB_ALIGN):
        self.context = context
        self.dims = dict(layers=layers, d=d, f=f, fs=fs, num_experts=num_experts, top_k=top_k)
        self.pool = ExpertPool(context, layers, num_experts, d, f, align)
        self.pool.fill_synthetic(seed)
        self.layers = []
        rng = np.random.default_rng(seed)
        self.norm_weights = []
        for l in range(layers):
            layer = MoEBlockLayer(context, self.pool, l, d, f, fs, num_experts, top_k)
            layer.fill_synthetic(seed * 1000 + l)
            self.layers.append(layer)
            w = (1.0 + 0.02 * rng.standard_normal(d)).astype(np.float32)
            self.norm_weights.append(torch.from_numpy(_bf16_bits(w).view(np.int16)).cuda())
        torch.cuda.synchronize()
        self.eps = eps
        self._build()

    def _build(self) -> None:
        n = len(self.layers)
        self._c_layers = (MoELayer * n)(*[l.c_struct() for l in self.layers])
        self._c_norms = (C.c_void_p * n)(*[w.data_ptr() for w in self.norm_weights])
        if getattr(self, "handle", None):
            self.context.lib.tf_stack_destroy(self.handle)
        handle = C.c_void_p()
        self.context.check(self.context.lib.tf_stack_create(self.context.handle, self._c_layers, self._c_norms, n,
                                                            self.eps, C.byref(handle)))
        self.handle = handle

    def set_logit_bias(self, bias: np.ndarray | None) -> None:
        for l in self.layers:
            l.set_logit_bias(bias)
        self._build()

    def workspace(self, max_tokens: int) -> Workspace:
        d = self.dims
        return Workspace(self.context, max_tokens, d["d"], d["f"], d["fs"], d["top_k"], d["num_experts"])

    def forward(self, hidden: torch.Tensor, tokens: int, ws: Workspace, stream=None) -> None:
        """hidden: fp16 [tokens, d] on the device, updated in place."""
        ctx = self.context
        ctx.check(ctx.lib.tf_stack_forward(self.handle, _stream(stream), _ptr(hidden), tokens, ws.handle))

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.context.lib.tf_stack_destroy(self.handle)
            self.handle = None
        self.pool.close()
