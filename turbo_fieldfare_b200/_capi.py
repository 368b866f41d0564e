"""ctypes binding of ``libtfcuda.so`` (declared in ``include/turbofieldfare_cuda.h``).

There is no CPU fallback and no JIT: if the in-tree shared library is missing
the import fails with an instruction to build it.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "_lib" / "libtfcuda.so"
HEADER_PATH = PKG.parent / "include" / "turbofieldfare_cuda.h"

TF_BF16, TF_FP16 = 0, 1
TF_MAX_TOP_K = 8

vp, u32, u64, i32, f32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int32, C.c_float


class ExpertOffsets(C.Structure):
    """tf_expert_offsets: nine byte offsets (MoEExpertOffsets, Kernels/MoE/MoE.swift:4-29)."""
    _fields_ = [(n, u32) for n in ("gate_w_off", "gate_s_off", "gate_b_off", "up_w_off", "up_s_off", "up_b_off",
                                   "down_w_off", "down_s_off", "down_b_off")]


class Projection(C.Structure):
    """tf_projection (SharedExpertProjection, Kernels/MoE/SharedExpertInt8.swift:9-31)."""
    _fields_ = [("weights", vp), ("weights_off", u64), ("scales", vp), ("scales_off", u64),
                ("biases", vp), ("biases_off", u64), ("rows", u32), ("cols", u32)]


class Pair(C.Structure):
    """tf_pair (PrefillTokenExpertPair, Kernels/Prefill/MoE/PrefillRouter.swift:5-28)."""
    _fields_ = [("token", u32), ("expert", u32), ("rank", u32), ("weight_bits_and_reserved", u32)]


class Group(C.Structure):
    _fields_ = [("expert", u32), ("pair_start", u32), ("pair_count", u32)]


class Tile(C.Structure):
    _fields_ = [("group_start", u32), ("group_count", u32), ("pair_start", u32), ("pair_count", u32)]


class MoELayer(C.Structure):
    """tf_moe_layer: device pointers and dimensions of one MoE block."""
    _fields_ = [("router", Projection), ("effective_scale", vp), ("per_expert_scale", vp), ("logit_bias", vp),
                ("pool_layer_base", vp), ("expert_stride", u64), ("offsets", ExpertOffsets),
                ("shared_gate", Projection), ("shared_up", Projection), ("shared_down", Projection),
                ("num_experts", u32), ("d", u32), ("f", u32), ("fs", u32), ("top_k", u32), ("shared_bits", u32)]


class GTurboInfo(C.Structure):
    """tf_gturbo_info: dimensions of an opened model directory."""
    _fields_ = [("version_major", u32), ("version_minor", u32), ("num_layers", u32), ("experts_per_layer", u32),
                ("top_k", u32), ("hidden_size", u32), ("moe_intermediate_size", u32), ("ffn_intermediate", u32),
                ("shared_expert_bits", u32), ("reserved", u32), ("expert_stride", u64), ("index_size", u64),
                ("resident_size", u64), ("entry_count", u64)]


class GTurboTensor(C.Structure):
    """tf_gturbo_tensor: one resident tensor, offsets relative to the resident payload."""
    _fields_ = [("offset", u64), ("size", u64), ("scale_offset", u64), ("scale_size", u64), ("bias_offset", u64),
                ("bias_size", u64), ("shape", u32 * 4), ("dtype", C.c_uint8), ("reserved", C.c_uint8 * 7)]


class StreamedParams(C.Structure):
    """tf_streamed_params: the 128-byte PrefillGroupedRoutedMoEStreamedParams
    (Kernels/Prefill/MoE/PrefillGroupedRoutedMoE.swift:104-183)."""
    _fields_ = ([(n, u32) for n in ("pair_start", "pair_count", "d", "routed_intermediate", "top_k", "hidden_stride_elements",
                                    "live_expert_count")] + [("local_expert", u32 * 16)] +
                [(n, u32) for n in ("gate_w_off", "gate_s_off", "gate_b_off", "up_w_off", "up_s_off", "up_b_off",
                                    "down_w_off", "down_s_off", "down_b_off")])


class DeviceRoutes(C.Structure):
    """tf_device_routes: device buffers of the grouped routing metadata."""
    _fields_ = [(n, vp) for n in ("sorted_pairs", "per_expert_offsets", "per_expert_counts", "groups",
                                  "chunk_group", "chunk_start", "counters")]


_PLANES = [vp, u64, vp, u64, vp, u64]   # weights, scales, biases with offsets

SIGNATURES = {
    "tf_abi_version": (C.c_int, []),
    "tf_context_create": (C.c_int, [C.c_int, C.POINTER(vp)]),
    "tf_context_destroy": (None, [vp]),
    "tf_last_error": (C.c_char_p, [vp]),
    "tf_context_set_step_trace": (C.c_int, [vp, vp, u32]),
    "tf_ep_unique_id": (C.c_int, [vp]),
    "tf_ep_create": (C.c_int, [vp, vp, C.c_int, C.c_int, C.POINTER(vp)]),
    "tf_ep_create_from_comm": (C.c_int, [vp, vp, C.c_int, C.c_int, C.POINTER(vp)]),
    "tf_ep_destroy": (None, [vp]),
    "tf_ep_rank": (C.c_int, [vp]),
    "tf_ep_world": (C.c_int, [vp]),
    "tf_ep_buffers_create": (C.c_int, [vp, u32, u32, u32, u32, u32, u32, C.c_int, C.POINTER(vp)]),
    "tf_ep_buffers_destroy": (None, [vp]),
    "tf_ep_buffers_mode": (C.c_int, [vp]),
    "tf_ep_buffers_workspace": (vp, [vp]),
    "tf_moe_block_forward_ep": (C.c_int, [vp, vp, C.POINTER(MoELayer), vp, vp, u32, vp]),
    "tf_stack_forward_ep": (C.c_int, [vp, vp, C.POINTER(MoELayer), C.POINTER(vp), u32, f32, vp, u32, vp]),
    "tf_context_set_single_launch_step": (C.c_int, [vp, C.c_int]),
    "tf_launch_count": (u64, [vp]),
    "tf_device_status": (C.c_int, [vp, C.POINTER(u32)]),
    "tf_int4_gemv": (C.c_int, [vp, vp, *_PLANES, vp, u64, vp, u64, u32, u32, C.c_int]),
    "tf_int4_gemv_batched": (C.c_int, [vp, vp, vp, u64, vp, u64, vp, u64, u64, vp, u64, u32, vp, u64, u32, u32, u32, u32, C.c_int]),
    "tf_int8_gemv": (C.c_int, [vp, vp, *_PLANES, vp, u64, vp, u64, u32, u32, C.c_int]),
    "tf_router_gemma4": (C.c_int, [vp, vp, *_PLANES, vp, vp, u64, vp, u64, vp, vp, vp, u32, u32, u32]),
    "tf_router_gemma4_block": (C.c_int, [vp, vp, *_PLANES, vp, u64, C.c_int, vp, u64, vp, u64, vp,
                                         vp, u64, vp, u64, vp, u32, u32, u32, u32, u32]),
    "tf_router_gemma4_block_grouped": (C.c_int, [vp, vp, *_PLANES, vp, u64, C.c_int, vp, u64, vp, u64, vp, vp, vp,
                                                 u32, u32, u32, u32, u32, C.POINTER(DeviceRoutes)]),
    "tf_moe_phase1": (C.c_int, [vp, vp, vp, C.POINTER(ExpertOffsets), vp, vp, u32, u32, u32]),
    "tf_moe_phase1_subset": (C.c_int, [vp, vp, vp, C.POINTER(ExpertOffsets), vp, vp, u32, u32, u32, vp, u32]),
    "tf_moe_phase2_reduce": (C.c_int, [vp, vp, vp, C.POINTER(ExpertOffsets), vp, vp, vp, vp, u32, u32, u32]),
    "tf_expert_table_from_indices": (C.c_int, [vp, vp, vp, u64, vp, u32, u32, vp]),
    "tf_shared_expert_int4": (C.c_int, [vp, vp, vp, u64, u64, C.POINTER(Projection), C.POINTER(Projection),
                                        C.POINTER(Projection), vp, u64, u64, vp, u64, u64, vp, u64, u64, vp, u64, u64]),
    "tf_make_token_expert_pairs": (C.c_int, [vp, vp, u32, u32, vp]),
    "tf_group_pairs": (C.c_int, [vp, u32, i32, i32, i32, i32, vp, u32, vp, vp, vp, vp, C.POINTER(u32), vp, C.POINTER(u32)]),
    "tf_group_routes_device": (C.c_int, [vp, vp, vp, vp, u32, u32, u32, C.POINTER(DeviceRoutes)]),
    "tf_grouped_moe_batched": (C.c_int, [vp, vp, vp, u64, u32, vp, u64, C.POINTER(ExpertOffsets), C.POINTER(DeviceRoutes),
                                         vp, vp, C.c_int, u32, u32, u32, u32]),
    "tf_grouped_moe_streamed": (C.c_int, [vp, vp, vp, u64, vp, u64, vp, u64, vp, u64, C.POINTER(vp), u32, vp, u32, C.POINTER(u32)]),
    "tf_moe_reduce_token_major": (C.c_int, [vp, vp, vp, C.c_int, vp, vp, u32, vp, u32, u32, u32, u32]),
    "tf_shared_expert_int8_block": (C.c_int, [vp, vp, vp, u64, u32, C.POINTER(Projection), C.POINTER(Projection),
                                              C.POINTER(Projection), vp, u64, u32, vp, u32]),
    "tf_shared_expert_int4_block": (C.c_int, [vp, vp, vp, u64, u32, C.POINTER(Projection), C.POINTER(Projection),
                                              C.POINTER(Projection), vp, u64, u32, vp, u32]),
    "tf_context_set_tensorcore_min_tokens": (C.c_int, [vp, u32]),
    "tf_context_set_shared_tensorcore_min_tokens": (C.c_int, [vp, u32]),
    "tf_context_set_router_tensorcore_min_rows": (C.c_int, [vp, u32]),
    "tf_context_set_ep_tensorcore_min_rows_per_expert": (C.c_int, [vp, u32]),
    "tf_int4_qmm": (C.c_int, [vp, vp, vp, u64, vp, u64, vp, u64, vp, u64, vp, u64, u32, u32, u32]),
    "tf_int4_qmm_with_path": (C.c_int, [vp, vp, vp, u64, vp, u64, vp, u64, vp, u64, vp, u64, u32, u32, u32, C.POINTER(C.c_int)]),
    "tf_pack_sorted_rows": (C.c_int, [vp, vp, vp, u32, C.POINTER(DeviceRoutes), u32, u32, u32, u32, vp, vp, vp]),
    "tf_grouped_moe_tensorcore": (C.c_int, [vp, vp, vp, u32, vp, u64, u32, C.POINTER(ExpertOffsets),
                                            C.POINTER(DeviceRoutes), vp, vp, u32, u32]),
    "tf_shared_expert_int4_tensorcore": (C.c_int, [vp, vp, vp, u32, C.POINTER(Projection), C.POINTER(Projection),
                                                   C.POINTER(Projection), vp, u32, vp, u32]),
    "tf_shared_expert_int4_block_noalloc": (C.c_int, [vp, vp, u64, u32, C.POINTER(Projection), C.POINTER(Projection),
                                                      C.POINTER(Projection), vp, u64, u32, u32, vp]),
    "tf_expert_pool_create": (C.c_int, [vp, u32, u32, u64, C.POINTER(ExpertOffsets), C.POINTER(vp)]),
    "tf_expert_pool_destroy": (None, [vp]),
    "tf_expert_pool_ptr": (vp, [vp, u32, u32]),
    "tf_expert_pool_bytes": (u64, [vp]),
    "tf_expert_pool_upload": (C.c_int, [vp, vp, u32, u32, vp, u64]),
    "tf_expert_pool_dims": (None, [vp, C.POINTER(u32), C.POINTER(u32), C.POINTER(u64)]),
    "tf_gturbo_open": (C.c_int, [C.c_char_p, C.POINTER(vp)]),
    "tf_gturbo_parse": (C.c_int, [vp, u64, vp, u64, vp, u64, C.POINTER(vp)]),
    "tf_gturbo_close": (None, [vp]),
    "tf_gturbo_get_info": (C.c_int, [vp, C.POINTER(GTurboInfo)]),
    "tf_gturbo_expert_offsets": (C.c_int, [vp, u32, C.POINTER(ExpertOffsets)]),
    "tf_gturbo_expert_location": (C.c_int, [vp, u32, u32, C.POINTER(C.c_char_p), C.POINTER(u64), C.POINTER(u64),
                                            C.POINTER(u32)]),
    "tf_gturbo_resident": (C.c_int, [vp, C.c_char_p, C.POINTER(GTurboTensor)]),
    "tf_gturbo_resident_name": (C.c_int, [vp, u64, C.POINTER(C.c_char_p)]),
    "tf_expert_pool_load_gturbo": (C.c_int, [vp, vp, vp, u32]),
    "tf_gturbo_model_load": (C.c_int, [vp, vp, vp, vp, C.POINTER(vp)]),
    "tf_gturbo_model_destroy": (None, [vp]),
    "tf_gturbo_model_layers": (C.POINTER(MoELayer), [vp, C.POINTER(u32)]),
    "tf_gturbo_model_resident_base": (vp, [vp]),
    "tf_fill_affine_synthetic": (C.c_int, [vp, vp, vp, vp, vp, u32, u32, u32, u64]),
    "tf_expert_pool_fill_synthetic": (C.c_int, [vp, vp, u64, u32, u32, u32, u32]),
    "tf_expert_pool_fill_synthetic_placed": (C.c_int, [vp, vp, u64, u32, u32, u32, vp]),
    "tf_ep_balanced_placement": (C.c_int, [vp, u32, u32, u32, vp]),
    "tf_workspace_create": (C.c_int, [vp, u32, u32, u32, u32, u32, u32, C.POINTER(vp)]),
    "tf_workspace_destroy": (None, [vp]),
    "tf_workspace_bytes": (u64, [vp]),
    "tf_workspace_indices": (vp, [vp]),
    "tf_workspace_weights": (vp, [vp]),
    "tf_workspace_routes": (C.POINTER(DeviceRoutes), [vp]),
    "tf_moe_block_forward": (C.c_int, [vp, vp, C.POINTER(MoELayer), vp, u32, vp, u32, u32, vp]),
    "tf_moe_block_forward_bf16": (C.c_int, [vp, vp, C.POINTER(MoELayer), vp, u32, vp, u32, u32, vp]),
    "tf_convert_rows": (C.c_int, [vp, vp, vp, C.c_int, u32, vp, C.c_int, u32, u32, u32]),
    "tf_stack_create": (C.c_int, [vp, C.POINTER(MoELayer), C.POINTER(vp), u32, f32, C.POINTER(vp)]),
    "tf_stack_destroy": (None, [vp]),
    "tf_stack_forward": (C.c_int, [vp, vp, vp, u32, vp]),
    "tf_residual_rmsnorm": (C.c_int, [vp, vp, vp, vp, vp, vp, u32, u32, f32]),
    "tf_ep_dispatch": (C.c_int, [vp, vp, C.POINTER(MoELayer), vp, u32, vp, u32, u32, vp, vp, vp, u32]),
    "tf_ep_experts": (C.c_int, [vp, vp, vp, u64, C.POINTER(ExpertOffsets), vp, vp, u32, u32, C.POINTER(DeviceRoutes), vp, vp, vp, u32, u32,
                                u32]),
    "tf_ep_experts_tensorcore": (C.c_int, [vp, vp, vp, u64, C.POINTER(ExpertOffsets), vp, vp, u32, u32, C.POINTER(DeviceRoutes),
                                           vp, vp, vp, vp, vp, vp, vp, vp, u32, u32]),
    "tf_ep_finish": (C.c_int, [vp, vp, C.POINTER(MoELayer), vp, u32, vp, vp, vp, vp]),
    "tf_ep_pack": (C.c_int, [vp, vp, vp, u64, u32, C.POINTER(DeviceRoutes), u32, u32, u32, u32, u32, u32, vp, vp, vp, u32]),
    "tf_ep_extract_ids": (C.c_int, [vp, vp, vp, u32, u32, u32, vp]),
    "tf_ep_combine": (C.c_int, [vp, vp, vp, vp, vp, vp, u32, vp, u32, u32, u32, u32]),
    "tf_rmsnorm": (C.c_int, [vp, vp, vp, u64, vp, u64, vp, u64, u32, u32, u32, f32, C.c_int]),
    "tf_peer_buffer_create": (C.c_int, [vp, u64, C.POINTER(vp)]),
    "tf_peer_buffer_destroy": (None, [vp]),
    "tf_peer_buffer_ptr": (vp, [vp]),
    "tf_peer_buffer_export": (C.c_int, [vp, vp]),
    "tf_peer_buffer_import": (C.c_int, [vp, vp, C.POINTER(vp)]),
    "tf_peer_buffer_release": (C.c_int, [vp, vp]),
    "tf_ep_peer_push": (C.c_int, [vp, vp, vp, u32, vp, u64, u32, u32, vp, u32, u32, u32, u32, u64, vp]),
    "tf_ep_peer_barrier": (C.c_int, [vp, vp, vp, u64, vp, u32, u32]),
    "tf_ep_pack_push": (C.c_int, [vp, vp, vp, u32, vp, u32, u32, u32, u32, u32, vp, u64, u32, vp, u32, u32, u32, u64, vp]),
    "tf_lm_head_greedy_int4": (C.c_int, [vp, vp, vp, u64, vp, u64, *_PLANES, vp, u32, u32, f32]),
    "tf_post_attn_setup": (C.c_int, [vp, vp, vp, u32, vp, u32, vp, u32, vp, u32, vp, u32, vp, vp, vp, u32, u32, f32]),
    "tf_layer_tail": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, f32, f32]),
}

_lib = None


def load() -> C.CDLL:
    """Load the in-tree library and attach the signatures. Raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m turbo_fieldfare_b200.build` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback for this library.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def declared_functions() -> list[str]:
    """Names of every function declared in the public header."""
    import re
    text = HEADER_PATH.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tf_[a-z0-9_]+)\s*\(", text)))
