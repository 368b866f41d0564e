"""Host-side mirror of the reference's operator classes over the C ABI.

Class and method names follow the Swift wrappers in
``Sources/TurboFieldfare/Kernels`` (``MoE.encodeRouterGemma4``,
``DequantInt4GEMV.encode`` ...). A ``torch.Tensor`` on the CUDA device stands in
for an ``MTLBuffer`` and a CUDA stream for the command buffer; every call only
enqueues work. Errors the reference raises as preconditions or thrown enums
arrive as :class:`TFError` carrying the C status code.

torch is used for device memory and streams only; no torch operator computes
anything on this path.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _capi
from ._capi import ExpertOffsets, Projection, TF_BF16, TF_FP16


class TFError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[tf_status {status}] {message}")
        self.status = status
        self.message = message


def _ptr(t) -> int | None:
    if t is None:
        return None
    if isinstance(t, torch.Tensor):
        return t.data_ptr()
    return int(t)


def _stream(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, torch.cuda.Stream):
        return stream.cuda_stream
    return int(stream)


class TurboContext:
    """Replaces ``MetalContext`` (Infrastructure/Metal/MetalContext.swift:51-214)."""

    def __init__(self, device: int = 0):
        self.lib = _capi.load()
        handle = C.c_void_p()
        status = self.lib.tf_context_create(device, C.byref(handle))
        if status != 0:
            raise TFError(status, self.lib.tf_last_error(None).decode())
        self.handle = handle
        self.device = device

    def check(self, status: int) -> None:
        if status != 0:
            raise TFError(status, self.lib.tf_last_error(self.handle).decode())

    def device_status(self) -> int:
        """Synchronise and return the device error word (0 = healthy); raises TFError when a kernel gave up a wait."""
        code = C.c_uint32(0)
        self.check(self.lib.tf_device_status(self.handle, C.byref(code)))
        return int(code.value)

    def set_tensorcore_min_tokens(self, tokens: int) -> None:
        """Blocks of at least ``tokens`` tokens run their expert GEMMs on the tensor cores (default 256)."""
        self.check(self.lib.tf_context_set_tensorcore_min_tokens(self.handle, tokens))

    def set_ep_tensorcore_min_rows_per_expert(self, rows: int) -> None:
        """Fixed-capacity expert-parallel buffers created afterwards run the expert phase on the tensor cores when the
        expected rows per local expert reach ``rows`` (off by default)."""
        self.check(self.lib.tf_context_set_ep_tensorcore_min_rows_per_expert(self.handle, rows))

    def set_shared_tensorcore_min_tokens(self, tokens: int) -> None:
        """The same threshold for a block's shared expert alone (default 256)."""
        self.check(self.lib.tf_context_set_shared_tensorcore_min_tokens(self.handle, tokens))

    def set_router_tensorcore_min_rows(self, rows: int) -> None:
        """Router calls over at least ``rows`` rows compute all logits on the tensor cores and re-check the candidates in
        the canonical order (default 256; 0xFFFFFFFF keeps the one-launch kernel)."""
        self.check(self.lib.tf_context_set_router_tensorcore_min_rows(self.handle, rows))

    def set_single_launch_step(self, enabled: bool) -> None:
        """One-token stack steps as one persistent launch (True) or layer by layer (False)."""
        self.check(self.lib.tf_context_set_single_launch_step(self.handle, 1 if enabled else 0))

    @property
    def launch_count(self) -> int:
        return int(self.lib.tf_launch_count(self.handle))

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.tf_context_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


@dataclass
class SharedExpertProjection:
    """(weights, scales, biases) buffers + byte offsets + shape (SharedExpertInt8.swift:9-31)."""
    weights: torch.Tensor
    scales: torch.Tensor
    biases: torch.Tensor
    rows: int
    cols: int
    weights_offset: int = 0
    scales_offset: int = 0
    biases_offset: int = 0

    def c_struct(self) -> Projection:
        return Projection(_ptr(self.weights), self.weights_offset, _ptr(self.scales), self.scales_offset,
                          _ptr(self.biases), self.biases_offset, self.rows, self.cols)


class DequantInt4GEMV:
    """``DequantInt4GEMV`` (Kernels/Quant/DequantInt4GEMV.swift:5-88)."""
    _fn = "tf_int4_gemv"

    def __init__(self, context: TurboContext):
        self.context = context

    def encode(self, weights, scales, biases, x, y, m: int, n: int, *, weights_offset=0, scales_offset=0,
               biases_offset=0, x_offset=0, y_offset=0, sb_dtype=TF_BF16, stream=None) -> None:
        ctx = self.context
        fn = getattr(ctx.lib, self._fn)
        ctx.check(fn(ctx.handle, _stream(stream), _ptr(weights), weights_offset, _ptr(scales), scales_offset,
                     _ptr(biases), biases_offset, _ptr(x), x_offset, _ptr(y), y_offset, m, n, sb_dtype))


    def encode_batched(self, weights, scales, biases, matrix_stride_bytes: int, x, y, m: int, n: int, count: int, *,
                       weights_offset=0, scales_offset=0, biases_offset=0, x_offset=0, x_stride_elements=0, y_offset=0,
                       y_stride_elements=None, sb_dtype=TF_BF16, stream=None) -> None:
        """``count`` GEMVs over matrices of one layout (planes ``matrix_stride_bytes`` apart) in one launch."""
        ctx = self.context
        ctx.check(ctx.lib.tf_int4_gemv_batched(ctx.handle, _stream(stream), _ptr(weights), weights_offset, _ptr(scales),
                                               scales_offset, _ptr(biases), biases_offset, matrix_stride_bytes, _ptr(x), x_offset,
                                               x_stride_elements, _ptr(y), y_offset, m if y_stride_elements is None else y_stride_elements,
                                               m, n, count, sb_dtype))


class DequantInt8GEMV(DequantInt4GEMV):
    """``DequantInt8GEMV`` (Kernels/Quant/DequantInt8GEMV.swift:16-82)."""
    _fn = "tf_int8_gemv"


class MoE:
    """``MoE`` (Kernels/MoE/MoE.swift:31-313): router + decode routed phases."""
    max_streamed_experts = 8

    def __init__(self, context: TurboContext):
        self.context = context

    def encode_router_gemma4(self, weights, scales, biases, hidden, effective_scale, per_expert_scale,
                             out_indices, out_weights, num_experts: int, d: int, top_k: int, *,
                             weights_offset=0, scales_offset=0, biases_offset=0, effective_scale_offset=0,
                             per_expert_scale_offset=0, out_logits=None, stream=None) -> None:
        ctx = self.context
        ctx.check(ctx.lib.tf_router_gemma4(
            ctx.handle, _stream(stream), _ptr(weights), weights_offset, _ptr(scales), scales_offset,
            _ptr(biases), biases_offset, _ptr(hidden), _ptr(effective_scale), effective_scale_offset,
            _ptr(per_expert_scale), per_expert_scale_offset, _ptr(out_indices), _ptr(out_weights),
            _ptr(out_logits), num_experts, d, top_k))

    def encode_routed_phase1(self, blobs, offsets: ExpertOffsets, x, acts, d: int, f: int, top_k: int, *, stream=None):
        ctx = self.context
        ctx.check(ctx.lib.tf_moe_phase1(ctx.handle, _stream(stream), _ptr(blobs), C.byref(offsets), _ptr(x),
                                        _ptr(acts), d, f, top_k))

    def encode_routed_phase1_subset(self, blobs, offsets: ExpertOffsets, x, acts, d: int, f: int, top_k: int,
                                    active_slots, active_count: int, *, stream=None):
        ctx = self.context
        ctx.check(ctx.lib.tf_moe_phase1_subset(ctx.handle, _stream(stream), _ptr(blobs), C.byref(offsets), _ptr(x),
                                               _ptr(acts), d, f, top_k, _ptr(active_slots), active_count))

    def encode_routed_phase2_reduce(self, blobs, offsets: ExpertOffsets, acts, routing_weights, residual, y,
                                    d: int, f: int, top_k: int, *, stream=None):
        ctx = self.context
        ctx.check(ctx.lib.tf_moe_phase2_reduce(ctx.handle, _stream(stream), _ptr(blobs), C.byref(offsets), _ptr(acts),
                                               _ptr(routing_weights), _ptr(residual), _ptr(y), d, f, top_k))

    def encode_expert_table(self, pool_layer_base, expert_stride: int, indices, count: int, num_experts: int,
                            blobs_out, *, stream=None):
        ctx = self.context
        ctx.check(ctx.lib.tf_expert_table_from_indices(ctx.handle, _stream(stream), _ptr(pool_layer_base),
                                                       expert_stride, _ptr(indices), count, num_experts,
                                                       _ptr(blobs_out)))


class SharedExpertInt4:
    """``SharedExpertInt4`` (Kernels/MoE/SharedExpertInt4.swift:21-95)."""

    def __init__(self, context: TurboContext):
        self.context = context

    def encode(self, x, gate: SharedExpertProjection, up: SharedExpertProjection, down: SharedExpertProjection, y,
               scratch_gate, scratch_up, scratch_act, *, x_offset=0, y_offset=0, scratch_gate_offset=0,
               scratch_up_offset=0, scratch_act_offset=0, stream=None) -> None:
        ctx = self.context
        nbytes = lambda t: t.numel() * t.element_size()
        g, u, dn = gate.c_struct(), up.c_struct(), down.c_struct()
        ctx.check(ctx.lib.tf_shared_expert_int4(
            ctx.handle, _stream(stream), _ptr(x), x_offset, nbytes(x), C.byref(g), C.byref(u), C.byref(dn),
            _ptr(y), y_offset, nbytes(y), _ptr(scratch_gate), scratch_gate_offset, nbytes(scratch_gate),
            _ptr(scratch_up), scratch_up_offset, nbytes(scratch_up), _ptr(scratch_act), scratch_act_offset,
            nbytes(scratch_act)))


class PrefillRouter:
    """``PrefillRouter`` (Kernels/Prefill/MoE/PrefillRouter.swift:30-112)."""

    def __init__(self, context: TurboContext):
        self.context = context

    def encode_gemma4_block(self, weights, scales, biases, hidden, effective_scale, per_expert_scale, out_indices,
                            out_weights, query_count: int, num_experts: int, d: int, top_k: int,
                            hidden_stride_elements: int, *, weights_offset=0, scales_offset=0, biases_offset=0,
                            hidden_offset=0, hidden_dtype=TF_FP16, effective_scale_offset=0,
                            per_expert_scale_offset=0, out_indices_offset=0, out_weights_offset=0,
                            logit_bias=None, out_logits=None, stream=None) -> None:
        ctx = self.context
        ctx.check(ctx.lib.tf_router_gemma4_block(
            ctx.handle, _stream(stream), _ptr(weights), weights_offset, _ptr(scales), scales_offset,
            _ptr(biases), biases_offset, _ptr(hidden), hidden_offset, hidden_dtype,
            _ptr(effective_scale), effective_scale_offset, _ptr(per_expert_scale), per_expert_scale_offset,
            _ptr(logit_bias), _ptr(out_indices), out_indices_offset, _ptr(out_weights), out_weights_offset,
            _ptr(out_logits), query_count, num_experts, d, top_k, hidden_stride_elements))

    def encode_gemma4_block_grouped(self, weights, scales, biases, hidden, effective_scale, per_expert_scale, out_indices,
                                    out_weights, query_count: int, num_experts: int, d: int, top_k: int,
                                    hidden_stride_elements: int, routes: "DeviceRoutes", *, weights_offset=0,
                                    scales_offset=0, biases_offset=0, hidden_offset=0, hidden_dtype=TF_FP16,
                                    effective_scale_offset=0, per_expert_scale_offset=0, logit_bias=None, stream=None) -> None:
        """Router and device grouping; one launch for blocks of at most 64 rows."""
        ctx = self.context
        ctx.check(ctx.lib.tf_router_gemma4_block_grouped(
            ctx.handle, _stream(stream), _ptr(weights), weights_offset, _ptr(scales), scales_offset,
            _ptr(biases), biases_offset, _ptr(hidden), hidden_offset, hidden_dtype,
            _ptr(effective_scale), effective_scale_offset, _ptr(per_expert_scale), per_expert_scale_offset,
            _ptr(logit_bias), _ptr(out_indices), _ptr(out_weights), query_count, num_experts, d, top_k,
            hidden_stride_elements, C.byref(routes.c_struct)))

    @staticmethod
    def make_token_expert_pairs(indices: np.ndarray, weights_f16_bits: np.ndarray, query_count: int, top_k: int):
        """Host arrays in, structured array of 16-byte pairs out (PrefillRouter.swift:91-111)."""
        lib = _capi.load()
        indices = np.ascontiguousarray(indices, dtype=np.uint32)
        weights = np.ascontiguousarray(weights_f16_bits, dtype=np.uint16)
        if indices.size != query_count * top_k:
            raise TFError(1, "indices count mismatch")
        if weights.size != query_count * top_k:
            raise TFError(1, "weights count mismatch")
        out = np.zeros(query_count * top_k, dtype=PAIR_DTYPE)
        status = lib.tf_make_token_expert_pairs(indices.ctypes.data, weights.ctypes.data, query_count, top_k,
                                                out.ctypes.data)
        if status:
            raise TFError(status, lib.tf_last_error(None).decode())
        return out


PAIR_DTYPE = np.dtype([("token", "<u4"), ("expert", "<u4"), ("rank", "<u4"), ("weight_bits", "<u4")])
GROUP_DTYPE = np.dtype([("expert", "<u4"), ("pair_start", "<u4"), ("pair_count", "<u4")])
TILE_DTYPE = np.dtype([("group_start", "<u4"), ("group_count", "<u4"), ("pair_start", "<u4"), ("pair_count", "<u4")])

GROUPING_ERROR_CASES = {
    101: "invalidQueryCount", 102: "invalidTopK", 103: "invalidNumExperts", 104: "invalidTileExpertCount",
    105: "pairCountMismatch", 106: "tokenOutOfRange", 107: "rankOutOfRange", 108: "expertOutOfRange",
    109: "duplicateTokenRank", 110: "expertSortKeyCountMismatch",
}


class PrefillMoEGroupingError(TFError):
    """``PrefillMoEGroupingError`` (PrefillMoEGrouping.swift:52-88)."""

    def __init__(self, status: int, message: str):
        super().__init__(status, message)
        self.case = GROUPING_ERROR_CASES.get(status)


@dataclass
class PrefillMoEGroupedRoutes:
    """``PrefillMoEGroupedRoutes`` (PrefillMoEGrouping.swift:33-50)."""
    sorted_pairs: np.ndarray
    per_expert_offsets: np.ndarray
    per_expert_counts: np.ndarray
    groups: np.ndarray
    tiles: np.ndarray
    query_count: int

    @property
    def max_pairs_per_expert(self) -> int:
        return int(self.groups["pair_count"].max()) if len(self.groups) else 0

    @property
    def max_pairs_per_tile(self) -> int:
        return int(self.tiles["pair_count"].max()) if len(self.tiles) else 0

    @property
    def max_live_experts_per_tile(self) -> int:
        return int(self.tiles["group_count"].max()) if len(self.tiles) else 0


class PrefillMoEGrouping:
    """``PrefillMoEGrouping`` (PrefillMoEGrouping.swift:90-193)."""

    @staticmethod
    def group_token_expert_pairs(pairs: np.ndarray, query_count: int, top_k: int, num_experts: int,
                                 tile_expert_count: int = 16, expert_sort_keys=None) -> PrefillMoEGroupedRoutes:
        lib = _capi.load()
        pairs = np.ascontiguousarray(pairs, dtype=PAIR_DTYPE)
        n = int(pairs.shape[0])
        sorted_out = np.zeros(max(n, 1), dtype=PAIR_DTYPE)
        offs = np.zeros(max(num_experts, 1), dtype=np.uint32)
        cnts = np.zeros(max(num_experts, 1), dtype=np.uint32)
        groups = np.zeros(max(n, 1), dtype=GROUP_DTYPE)
        tiles = np.zeros(max(n, 1), dtype=TILE_DTYPE)
        ng, nt = C.c_uint32(0), C.c_uint32(0)
        keys = None if expert_sort_keys is None else np.ascontiguousarray(expert_sort_keys, dtype=np.uint64)
        status = lib.tf_group_pairs(pairs.ctypes.data, n, query_count, top_k, num_experts, tile_expert_count,
                                    None if keys is None else keys.ctypes.data, 0 if keys is None else keys.shape[0],
                                    sorted_out.ctypes.data, offs.ctypes.data, cnts.ctypes.data, groups.ctypes.data,
                                    C.byref(ng), tiles.ctypes.data, C.byref(nt))
        if status:
            raise PrefillMoEGroupingError(status, lib.tf_last_error(None).decode())
        return PrefillMoEGroupedRoutes(sorted_out[:n], offs[:num_experts], cnts[:num_experts],
                                       groups[:ng.value], tiles[:nt.value], query_count)


class RMSNorm:
    """``RMSNorm`` / ``PrefillRMSNorm`` (Metal/Primitives/rmsnorm.metal:32-93,153-175)."""

    def __init__(self, context: TurboContext):
        self.context = context

    def encode(self, x, weight, y, rows: int, d: int, stride_elements: int | None = None, eps: float = 1e-6,
               act_dtype=TF_FP16, *, x_offset=0, weight_offset=0, y_offset=0, stream=None):
        ctx = self.context
        ctx.check(ctx.lib.tf_rmsnorm(ctx.handle, _stream(stream), _ptr(x), x_offset, _ptr(weight), weight_offset,
                                     _ptr(y), y_offset, rows, d, d if stride_elements is None else stride_elements,
                                     eps, act_dtype))


class LMHeadChainInt4:
    """``LMHeadChainInt4.encodeGreedyDecode`` (Kernels/Fusions/LMHeadChainInt4.swift:53-135): final RMSNorm, tied int4
    LM head, greedy token. ``out_token`` is a device uint32."""

    def __init__(self, context: TurboContext):
        self.context = context

    def encode_greedy_decode(self, hidden, norm_weight, weights, scales, biases, out_token, d: int, vocab: int,
                             rms_eps: float = 1e-6, *, hidden_offset=0, norm_offset=0, weights_offset=0, scales_offset=0,
                             biases_offset=0, stream=None):
        ctx = self.context
        ctx.check(ctx.lib.tf_lm_head_greedy_int4(ctx.handle, _stream(stream), _ptr(hidden), hidden_offset,
                                                 _ptr(norm_weight), norm_offset, _ptr(weights), weights_offset,
                                                 _ptr(scales), scales_offset, _ptr(biases), biases_offset,
                                                 _ptr(out_token), d, vocab, rms_eps))


class FusedPostAttentionSetup:
    """``FusedPostAttentionSetup`` / ``PrefillPostAttentionSetup`` (Kernels/Fusions/FusedPostAttentionSetup.swift:26-60;
    Kernels/Prefill/Epilogues/PrefillPostAttentionSetup.swift): the three-way norm in front of the feed-forward block."""

    def __init__(self, context: TurboContext):
        self.context = context

    def encode(self, hidden, attn, dense_x, routed_x, router_x, post_attention_weight, pre_ffn_weight, pre_ffn2_weight,
               d: int, eps: float = 1e-6, *, rows: int = 1, hidden_stride: int | None = None, attn_stride: int | None = None,
               dense_stride: int | None = None, routed_stride: int | None = None, router_stride: int | None = None,
               stream=None):
        ctx = self.context
        st = lambda v: d if v is None else v
        ctx.check(ctx.lib.tf_post_attn_setup(ctx.handle, _stream(stream), _ptr(hidden), st(hidden_stride), _ptr(attn),
                                             st(attn_stride), _ptr(dense_x), st(dense_stride), _ptr(routed_x),
                                             st(routed_stride), _ptr(router_x), st(router_stride),
                                             _ptr(post_attention_weight), _ptr(pre_ffn_weight), _ptr(pre_ffn2_weight),
                                             rows, d, eps))


class FusedLayerTail:
    """``FusedLayerTail`` / ``PrefillLayerTail`` (Metal/Fusions/fused.metal:271-375)."""

    def __init__(self, context: TurboContext):
        self.context = context

    def encode(self, h2, h1, hidden, w_postffn2, w_postffn, rows: int, d: int, stride_elements: int | None = None,
               eps: float = 1e-6, layer_scalar: float = 1.0, *, stream=None):
        ctx = self.context
        ctx.check(ctx.lib.tf_layer_tail(ctx.handle, _stream(stream), _ptr(h2), _ptr(h1), _ptr(hidden), _ptr(w_postffn2),
                                        _ptr(w_postffn), rows, d, d if stride_elements is None else stride_elements,
                                        eps, layer_scalar))


class DeviceRoutes:
    """Device buffers for the grouped routing metadata (``tf_device_routes``). Replaces the
    CPU-built ``PrefillMoEGroupedRoutes`` + ``makeStreamedMetadataBuffers``
    (Kernels/Prefill/MoE/PrefillGroupedRoutedMoE.swift:368-384)."""

    def __init__(self, max_tokens: int, top_k: int, num_experts: int, device="cuda"):
        n = max_tokens * top_k
        i32 = dict(dtype=torch.int32, device=device)
        self.max_tokens, self.top_k, self.num_experts = max_tokens, top_k, num_experts
        self.sorted_pairs = torch.zeros(max(n, 1) * 4, **i32)
        self.per_expert_offsets = torch.zeros(num_experts, **i32)
        self.per_expert_counts = torch.zeros(num_experts, **i32)
        self.groups = torch.zeros(num_experts * 3, **i32)
        self.chunk_group = torch.zeros(n // 8 + num_experts + 1, **i32)
        self.chunk_start = torch.zeros(num_experts, **i32)
        self.counters = torch.zeros(4, **i32)
        self.c_struct = _capi.DeviceRoutes(*[_ptr(t) for t in (self.sorted_pairs, self.per_expert_offsets,
                                                               self.per_expert_counts, self.groups, self.chunk_group,
                                                               self.chunk_start, self.counters)])

    def to_host(self, query_count: int) -> PrefillMoEGroupedRoutes:
        n = query_count * self.top_k
        counters = self.counters.cpu().numpy().view(np.uint32)
        ng = int(counters[0])
        return PrefillMoEGroupedRoutes(
            self.sorted_pairs.cpu().numpy().view(np.uint32)[:n * 4].copy().view(PAIR_DTYPE),
            self.per_expert_offsets.cpu().numpy().view(np.uint32), self.per_expert_counts.cpu().numpy().view(np.uint32),
            self.groups.cpu().numpy().view(np.uint32)[:ng * 3].copy().view(GROUP_DTYPE), np.zeros(0, dtype=TILE_DTYPE),
            query_count)


class PrefillGroupedRoutedMoE:
    """``PrefillGroupedRoutedMoE`` (Kernels/Prefill/MoE/PrefillGroupedRoutedMoE.swift:339-463) over
    HBM-resident experts, with the grouping done on the device."""

    def __init__(self, context: TurboContext):
        self.context = context

    def encode_group_routes(self, indices, weights, query_count: int, top_k: int, num_experts: int,
                            routes: DeviceRoutes, *, stream=None):
        ctx = self.context
        ctx.check(ctx.lib.tf_group_routes_device(ctx.handle, _stream(stream), _ptr(indices), _ptr(weights),
                                                 query_count, top_k, num_experts, C.byref(routes.c_struct)))

    def encode_streamed_batched(self, hidden, pool_layer_base, expert_stride: int, offsets: ExpertOffsets,
                                routes: DeviceRoutes, acts_scratch, route_partials, query_count: int, d: int, f: int,
                                top_k: int, *, hidden_offset=0, hidden_stride_elements=None, partials_f32=False,
                                stream=None):
        ctx = self.context
        ctx.check(ctx.lib.tf_grouped_moe_batched(
            ctx.handle, _stream(stream), _ptr(hidden), hidden_offset,
            d if hidden_stride_elements is None else hidden_stride_elements, _ptr(pool_layer_base), expert_stride,
            C.byref(offsets), C.byref(routes.c_struct), _ptr(acts_scratch), _ptr(route_partials),
            1 if partials_f32 else 0, query_count, d, f, top_k))


    def encode_pack_sorted_rows(self, hidden, routes: DeviceRoutes, query_count: int, top_k: int, num_experts: int, d: int,
                                x_sorted, row_expert_ids, inverse_perm, *, hidden_stride_elements=None, stream=None):
        """Gather every pair's hidden row into expert order for the tensor-core path (``tf_pack_sorted_rows``)."""
        ctx = self.context
        ctx.check(ctx.lib.tf_pack_sorted_rows(
            ctx.handle, _stream(stream), _ptr(hidden), d if hidden_stride_elements is None else hidden_stride_elements,
            C.byref(routes.c_struct), query_count, top_k, num_experts, d, _ptr(x_sorted), _ptr(row_expert_ids),
            _ptr(inverse_perm)))

    def encode_tensorcore(self, x_sorted, x_rows: int, pool_layer_base, expert_stride: int, num_experts: int,
                          offsets: ExpertOffsets, routes: DeviceRoutes, acts_scratch, out_rows, d: int, f: int, *,
                          stream=None):
        """Same operator on the tcgen05 tensor cores over expert-sorted rows (``tf_grouped_moe_tensorcore``)."""
        ctx = self.context
        ctx.check(ctx.lib.tf_grouped_moe_tensorcore(
            ctx.handle, _stream(stream), _ptr(x_sorted), x_rows, _ptr(pool_layer_base), expert_stride, num_experts,
            C.byref(offsets), C.byref(routes.c_struct), _ptr(acts_scratch), _ptr(out_rows), d, f))


class MPPPrefillInt4QMM:
    """``MPPPrefillInt4QMM`` (Kernels/TensorCore/MPPPrefillInt4QMM.swift:4-79): Y[M,N] = X[M,K] . deq4(W[N,K])^T with
    the weight tile staged as half and multiplied on the matrix unit (tcgen05 here, TensorOps there)."""

    def __init__(self, context: TurboContext):
        self.context = context

    def encode(self, weights, scales, biases, x, y, m: int, n: int, k: int, *, weights_offset=0, scales_offset=0,
               biases_offset=0, x_offset=0, y_offset=0, stream=None):
        """Returns the path that ran: ``"affine-threadgroup-f16"`` (tensor cores), ``"cuda-cores"`` (planes off the
        16-byte grid or N % 8 != 0) or ``"unavailable"`` (outside the reference's guard; nothing launched)."""
        ctx = self.context
        path = C.c_int(0)
        ctx.check(ctx.lib.tf_int4_qmm_with_path(ctx.handle, _stream(stream), _ptr(weights), weights_offset, _ptr(scales),
                                                scales_offset, _ptr(biases), biases_offset, _ptr(x), x_offset, _ptr(y),
                                                y_offset, m, n, k, C.byref(path)))
        return self.PATHS[path.value]

    PATHS = ("unavailable", "affine-threadgroup-f16", "cuda-cores")


class PrefillMoE:
    """``PrefillMoE`` (Kernels/Prefill/MoE/PrefillMoE.swift:4-40)."""

    def __init__(self, context: TurboContext):
        self.context = context

    def encode_reduce_token_major(self, route_partials, route_weights, h2, query_count: int, top_k: int, d: int, *,
                                  residual=None, residual_stride=None, h2_stride=None, partials_f32=False, stream=None):
        ctx = self.context
        ctx.check(ctx.lib.tf_moe_reduce_token_major(
            ctx.handle, _stream(stream), _ptr(route_partials), 1 if partials_f32 else 0, _ptr(route_weights),
            _ptr(residual), d if residual_stride is None else residual_stride, _ptr(h2),
            d if h2_stride is None else h2_stride, query_count, top_k, d))


class PrefillSharedExpert:
    """``PrefillSharedExpert`` (Kernels/Prefill/MoE/PrefillSharedExpert.swift:4-60), batched over rows."""

    def __init__(self, context: TurboContext):
        self.context = context

    def encode_block(self, x, gate: SharedExpertProjection, up: SharedExpertProjection, down: SharedExpertProjection,
                     y, scratch_act, rows: int, *, x_offset=0, x_stride=None, y_offset=0, y_stride=None, stream=None):
        ctx = self.context
        g, u, dn = gate.c_struct(), up.c_struct(), down.c_struct()
        ctx.check(ctx.lib.tf_shared_expert_int4_block(
            ctx.handle, _stream(stream), _ptr(x), x_offset, gate.cols if x_stride is None else x_stride,
            C.byref(g), C.byref(u), C.byref(dn), _ptr(y), y_offset, gate.cols if y_stride is None else y_stride,
            _ptr(scratch_act), rows))

    def encode_block_tensorcore(self, x, gate: SharedExpertProjection, up: SharedExpertProjection,
                                down: SharedExpertProjection, y, scratch_act, rows: int, *, x_stride=None, y_stride=None,
                                stream=None):
        """The block on the tcgen05 tensor cores (``tf_shared_expert_int4_tensorcore``), for prefill-sized blocks."""
        ctx = self.context
        g, u, dn = gate.c_struct(), up.c_struct(), down.c_struct()
        ctx.check(ctx.lib.tf_shared_expert_int4_tensorcore(
            ctx.handle, _stream(stream), _ptr(x), gate.cols if x_stride is None else x_stride,
            C.byref(g), C.byref(u), C.byref(dn), _ptr(y), gate.cols if y_stride is None else y_stride,
            _ptr(scratch_act), rows))
