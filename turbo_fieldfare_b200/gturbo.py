"""`.gturbo` model directories over the C ABI: open, inspect, upload into HBM.

Host-side mirror of the reference's readers: ``ManifestReader`` (Infrastructure/ModelIO/ManifestReader.swift:64-152),
``PackedExpertsLayoutReader`` (Infrastructure/ModelIO/PackedExpertsLayout.swift:57-119), ``ResidentIndexReader``
(Infrastructure/ModelIO/ResidentIndex.swift:44-140), ``Model.resident(name:)`` (Runtime/Inference/Model.swift:195-233)
and ``Model.routedExpertOffsets`` (Runtime/Inference/ModelExpertIO.swift:21-40). Parsing needs no GPU; the upload
replaces the pread streamer with one copy of every expert blob into the expert pool.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

from . import _capi
from ._capi import ExpertOffsets, GTurboInfo, GTurboTensor, MoELayer

DTYPE_NAMES = {0: "u32", 1: "bf16", 2: "fp16", 3: "fp32"}     # GTurboFormatV1.DType


class GTurboError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[tf_status {status}] {message}")
        self.status = status
        self.message = message


@dataclass(frozen=True)
class ResidentTensor:
    """Payload-relative view of one resident tensor (``TensorView`` of the reference)."""
    name: str
    dtype: str
    offset: int
    size: int
    scale_offset: int
    scale_size: int
    bias_offset: int
    bias_size: int
    shape: tuple


@dataclass(frozen=True)
class ExpertLocation:
    file: str
    offset: int
    size: int
    physical_rank: int


class GTurboDirectory:
    """An opened (parsed and validated) model directory."""

    def __init__(self, handle, lib):
        self._handle, self._lib = handle, lib
        info = GTurboInfo()
        self._check(lib.tf_gturbo_get_info(handle, C.byref(info)))
        self.info = info

    @classmethod
    def open(cls, directory: str | os.PathLike) -> "GTurboDirectory":
        lib = _capi.load()
        handle = C.c_void_p()
        status = lib.tf_gturbo_open(os.fsencode(directory), C.byref(handle))
        if status != 0:
            raise GTurboError(status, lib.tf_last_error(None).decode())
        return cls(handle, lib)

    @classmethod
    def parse(cls, manifest_json: bytes, layout_json: bytes, resident_index: bytes) -> "GTurboDirectory":
        """From memory: the two JSON documents and at least the index region of ``model_weights.bin``."""
        lib = _capi.load()
        handle = C.c_void_p()
        status = lib.tf_gturbo_parse(manifest_json, len(manifest_json), layout_json, len(layout_json),
                                     resident_index, len(resident_index), C.byref(handle))
        if status != 0:
            raise GTurboError(status, lib.tf_last_error(None).decode())
        return cls(handle, lib)

    def _check(self, status: int) -> None:
        if status != 0:
            raise GTurboError(status, self._lib.tf_last_error(None).decode())

    @property
    def handle(self):
        return self._handle

    def expert_offsets(self, layer: int) -> ExpertOffsets:
        out = ExpertOffsets()
        self._check(self._lib.tf_gturbo_expert_offsets(self._handle, layer, C.byref(out)))
        return out

    def expert(self, layer: int, expert: int) -> ExpertLocation:
        file, off, size, rank = C.c_char_p(), C.c_uint64(), C.c_uint64(), C.c_uint32()
        self._check(self._lib.tf_gturbo_expert_location(self._handle, layer, expert, C.byref(file), C.byref(off),
                                                        C.byref(size), C.byref(rank)))
        return ExpertLocation(file.value.decode(), off.value, size.value, rank.value)

    def resident(self, name: str) -> ResidentTensor:
        t = GTurboTensor()
        self._check(self._lib.tf_gturbo_resident(self._handle, name.encode(), C.byref(t)))
        return ResidentTensor(name, DTYPE_NAMES[t.dtype], t.offset, t.size, t.scale_offset, t.scale_size,
                              t.bias_offset, t.bias_size, tuple(t.shape))

    def resident_names(self) -> list[str]:
        names = []
        for k in range(self.info.entry_count):
            p = C.c_char_p()
            self._check(self._lib.tf_gturbo_resident_name(self._handle, k, C.byref(p)))
            names.append(p.value.decode())
        return names

    def close(self) -> None:
        if getattr(self, "_handle", None):
            self._lib.tf_gturbo_close(self._handle)
            self._handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class GTurboModel:
    """Every routed expert and the resident payload of a model directory in HBM, as ``tf_moe_layer`` records.

    Needs a GPU: creates the expert pool (``layers x experts x stride`` bytes), copies each blob to its logical
    slot and uploads ``model_weights.bin``'s payload."""

    def __init__(self, context, directory: GTurboDirectory, stream=None):
        import torch
        from .kernels import _stream
        self.context, self.directory = context, directory
        lib, info = context.lib, directory.info
        self.offsets = directory.expert_offsets(0)
        pool = C.c_void_p()
        context.check(lib.tf_expert_pool_create(context.handle, info.num_layers, info.experts_per_layer, info.expert_stride,
                                                C.byref(self.offsets), C.byref(pool)))
        self.pool = pool
        self.model = None
        try:
            status = lib.tf_expert_pool_load_gturbo(pool, _stream(stream), directory.handle, 0)
            if status != 0:
                raise GTurboError(status, lib.tf_last_error(None).decode())
            model = C.c_void_p()
            status = lib.tf_gturbo_model_load(context.handle, _stream(stream), directory.handle, pool, C.byref(model))
            if status != 0:
                raise GTurboError(status, lib.tf_last_error(None).decode())
            self.model = model
        except Exception:
            self.close()
            raise
        count = C.c_uint32()
        self._layers = lib.tf_gturbo_model_layers(self.model, C.byref(count))
        self.layer_count = int(count.value)
        torch.cuda.synchronize()

    def layer(self, index: int) -> MoELayer:
        if not 0 <= index < self.layer_count:
            raise IndexError(index)
        return self._layers[index]

    def expert_ptr(self, layer: int, expert: int) -> int:
        return self.context.lib.tf_expert_pool_ptr(self.pool, layer, expert)

    @property
    def resident_base(self) -> int:
        return self.context.lib.tf_gturbo_model_resident_base(self.model)

    def block_forward(self, layer: int, x, y, tokens: int, workspace, stream=None) -> None:
        """One MoE block of the loaded model: ``y = shared(x) + sum_r w_r routed_r(x)`` (fp16 rows of ``d`` elements)."""
        from .kernels import _ptr, _stream
        ctx, rec = self.context, self.layer(layer)
        ctx.check(ctx.lib.tf_moe_block_forward(ctx.handle, _stream(stream), C.byref(rec), _ptr(x), rec.d, _ptr(y), rec.d,
                                               tokens, workspace.handle))

    def close(self) -> None:
        lib = self.context.lib
        if getattr(self, "model", None):
            lib.tf_gturbo_model_destroy(self.model)
            self.model = None
        if getattr(self, "pool", None):
            lib.tf_expert_pool_destroy(self.pool)
            self.pool = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
