"""ctypes/numpy face of the CPU oracle (``tf_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``. The
product package never imports it.

All 16-bit float tensors are carried as ``numpy.uint16`` bit patterns so that
nothing depends on numpy's own float16 rounding.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libtforacle.so"


def build(force: bool = False) -> Path:
    """Compile the C restatement with the Makefile beside it."""
    src = _HERE / "tf_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        env = dict(os.environ)
        env.pop("CC", None)
        subprocess.run(["make", "-C", str(_HERE)], check=True, env=env,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(str(_LIB_PATH))
        _declare(_lib)
    return _lib


def _p(a: np.ndarray | None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle wants contiguous arrays"
    return a.ctypes.data_as(C.c_void_p)


class ExpertOffsets(C.Structure):
    """Nine byte offsets into an expert blob (Kernels/MoE/MoE.swift:4-29)."""
    _fields_ = [(n, C.c_uint32) for n in
                ("gate_w", "gate_s", "gate_b", "up_w", "up_s", "up_b", "down_w", "down_s", "down_b")]


PAIR_DTYPE = np.dtype([("token", "<u4"), ("expert", "<u4"), ("rank", "<u4"), ("weight_bits", "<u4")])
GROUP_DTYPE = np.dtype([("expert", "<u4"), ("pair_start", "<u4"), ("pair_count", "<u4")])
TILE_DTYPE = np.dtype([("group_start", "<u4"), ("group_count", "<u4"), ("pair_start", "<u4"), ("pair_count", "<u4")])


def _declare(l: C.CDLL) -> None:
    vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_int64, C.c_float
    l.tfo_bf16_bits.restype = C.c_uint16
    l.tfo_bf16_bits.argtypes = [f32]
    l.tfo_bf16_to_float.restype = f32
    l.tfo_bf16_to_float.argtypes = [C.c_uint16]
    l.tfo_f32_to_f16.restype = C.c_uint16
    l.tfo_f32_to_f16.argtypes = [f32]
    l.tfo_f16_to_f32.restype = f32
    l.tfo_f16_to_f32.argtypes = [C.c_uint16]
    for name in ("tfo_f32_to_f16_array", "tfo_f16_to_f32_array", "tfo_f32_to_bf16_array", "tfo_bf16_to_f32_array"):
        getattr(l, name).restype = None
        getattr(l, name).argtypes = [vp, vp, i64]
    l.tfo_splitmix64_next.restype = C.c_uint64
    l.tfo_splitmix64_next.argtypes = [C.POINTER(C.c_uint64)]
    l.tfo_uniform.restype = f32
    l.tfo_uniform.argtypes = [C.POINTER(C.c_uint64), f32, f32]
    l.tfo_uniform_fill.restype = None
    l.tfo_uniform_fill.argtypes = [C.POINTER(C.c_uint64), f32, f32, vp, i64]
    l.tfo_seedtree_key.restype = C.c_uint64
    l.tfo_seedtree_key.argtypes = [C.c_uint64, C.c_char_p]
    for name in ("tfo_quantize_int4_affine", "tfo_quantize_int8_affine"):
        getattr(l, name).restype = None
        getattr(l, name).argtypes = [vp, i32, vp, vp, vp]
    for name in ("tfo_dequantize_int4_affine", "tfo_dequantize_int8_affine"):
        getattr(l, name).restype = None
        getattr(l, name).argtypes = [vp, vp, vp, i32, i32, vp]
    l.tfo_affine_gemv_ref.restype = None
    l.tfo_affine_gemv_ref.argtypes = [vp, vp, vp, i32, vp, vp, i32, i32, i32, i32]
    for name in ("tfo_int4_gemv_kernel_order", "tfo_int8_gemv_kernel_order"):
        getattr(l, name).restype = None
        getattr(l, name).argtypes = [vp, vp, vp, i32, vp, vp, vp, i32, i32]
    l.tfo_router_logits.restype = None
    l.tfo_router_logits.argtypes = [vp, vp, vp, vp, i64, vp, vp, i32, i32, i32]
    l.tfo_router_logits_f64.restype = None
    l.tfo_router_logits_f64.argtypes = [vp, vp, vp, vp, i64, vp, vp, i32, i32, i32]
    l.tfo_router_select.restype = None
    l.tfo_router_select.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32]
    l.tfo_router_select_sorted.restype = None
    l.tfo_router_select_sorted.argtypes = [vp, vp, vp, vp, i32, i32]
    l.tfo_gelu_tanh.restype = f32
    l.tfo_gelu_tanh.argtypes = [f32]
    l.tfo_moe_routed_decode.restype = None
    l.tfo_moe_routed_decode.argtypes = [vp, C.POINTER(ExpertOffsets), vp, vp, vp, vp, vp, vp, i32, i32, i32, i32]
    l.tfo_shared_expert_int4.restype = None
    l.tfo_shared_expert_int4.argtypes = [vp] * 9 + [vp, vp, vp, i32, i32, i32]
    l.tfo_moe_reduce_token_major.restype = None
    l.tfo_moe_reduce_token_major.argtypes = [vp, vp, vp, i32, i32, i32]
    l.tfo_make_token_expert_pairs.restype = None
    l.tfo_make_token_expert_pairs.argtypes = [vp, vp, i32, i32, vp]
    l.tfo_group_pairs.restype = i32
    l.tfo_group_pairs.argtypes = [vp, i32, i32, i32, i32, i32, vp, i32, vp, vp, vp, vp,
                                  C.POINTER(i32), vp, C.POINTER(i32)]
    l.tfo_grouped_moe_pairs.restype = None
    l.tfo_grouped_moe_pairs.argtypes = [vp, i64, C.POINTER(ExpertOffsets), vp, i64, i32, vp, i32, vp, i32, i32, i32]
    l.tfo_int4_qmm_ref.restype = None
    l.tfo_int4_qmm_ref.argtypes = [vp, vp, vp, vp, i32, vp, i32, i32, i32]
    l.tfo_rmsnorm.restype = None
    l.tfo_rmsnorm.argtypes = [vp, vp, vp, i32, i32, i64, f32]
    l.tfo_layer_tail.restype = None
    l.tfo_layer_tail.argtypes = [vp, vp, vp, vp, vp, i32, i32, i64, f32, f32]
    l.tfo_num_threads.restype = i32
    l.tfo_set_num_threads.argtypes = [i32]


# ---------------------------------------------------------------------------
# conversions
# ---------------------------------------------------------------------------

def f32_to_f16(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().tfo_f32_to_f16_array(_p(a), _p(out), a.size)
    return out


def f16_to_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, dtype=np.float32)
    lib().tfo_f16_to_f32_array(_p(a), _p(out), a.size)
    return out


def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().tfo_f32_to_bf16_array(_p(a), _p(out), a.size)
    return out


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, dtype=np.float32)
    lib().tfo_bf16_to_f32_array(_p(a), _p(out), a.size)
    return out


# ---------------------------------------------------------------------------
# PRNG (SplitMix64.swift / SeedTree.swift)
# ---------------------------------------------------------------------------

class SplitMix64:
    def __init__(self, seed: int):
        self._state = C.c_uint64(seed & 0xFFFFFFFFFFFFFFFF)

    def next(self) -> int:
        return int(lib().tfo_splitmix64_next(C.byref(self._state)))

    def uniform(self, lo: float, hi: float) -> float:
        return float(lib().tfo_uniform(C.byref(self._state), lo, hi))

    def uniform_array(self, lo: float, hi: float, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        lib().tfo_uniform_fill(C.byref(self._state), lo, hi, _p(out), n)
        return out


class SeedTree:
    def __init__(self, root: int):
        self.root = root & 0xFFFFFFFFFFFFFFFF

    def key(self, label: str) -> SplitMix64:
        return SplitMix64(int(lib().tfo_seedtree_key(self.root, label.encode("utf-8"))))


# ---------------------------------------------------------------------------
# quantisers
# ---------------------------------------------------------------------------

@dataclass
class AffineMatrix:
    """Row-major affine-quantised matrix: packed codes + 16-bit scale/bias planes."""
    packed: np.ndarray   # uint8 [m, n/2] (4-bit) or [m, n] (8-bit)
    scales: np.ndarray   # uint16 [m, n/64]
    biases: np.ndarray   # uint16 [m, n/64]
    bits: int
    n: int
    sb_dtype: int = 0    # 0 bf16, 1 fp16

    @property
    def m(self) -> int:
        return self.packed.shape[0]


def quantize_rows(rows: np.ndarray, bits: int) -> AffineMatrix:
    rows = np.ascontiguousarray(rows, dtype=np.float32)
    m, n = rows.shape
    assert n % 64 == 0
    packed = np.zeros((m, n // 2 if bits == 4 else n), dtype=np.uint8)
    scales = np.zeros((m, n // 64), dtype=np.uint16)
    biases = np.zeros((m, n // 64), dtype=np.uint16)
    fn = lib().tfo_quantize_int4_affine if bits == 4 else lib().tfo_quantize_int8_affine
    for r in range(m):
        fn(_p(rows[r]), n, _p(packed[r]), _p(scales[r]), _p(biases[r]))
    return AffineMatrix(packed, scales, biases, bits, n)


def dequantize(mat: AffineMatrix) -> np.ndarray:
    out = np.empty((mat.m, mat.n), dtype=np.float32)
    fn = lib().tfo_dequantize_int4_affine if mat.bits == 4 else lib().tfo_dequantize_int8_affine
    for r in range(mat.m):
        fn(_p(mat.packed[r]), _p(mat.scales[r]), _p(mat.biases[r]), mat.sb_dtype, mat.n, _p(out[r]))
    return out


# ---------------------------------------------------------------------------
# GEMV
# ---------------------------------------------------------------------------

def gemv_ref(mat: AffineMatrix, x_f32: np.ndarray, acc: str = "f64") -> np.ndarray:
    """Dequantise-then-dot reference (DequantInt4Gemv.swift:13-42)."""
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    y = np.empty(mat.m, dtype=np.float32)
    lib().tfo_affine_gemv_ref(_p(mat.packed), _p(mat.scales), _p(mat.biases), mat.sb_dtype,
                              _p(x), _p(y), mat.m, mat.n, mat.bits, 0 if acc == "f64" else 1)
    return y


def gemv_kernel_order(mat: AffineMatrix, x_f16: np.ndarray):
    """The reference kernels' group-factored lane order; returns (y_f16 bits, y_f32)."""
    x = np.ascontiguousarray(x_f16, dtype=np.uint16)
    y16 = np.empty(mat.m, dtype=np.uint16)
    y32 = np.empty(mat.m, dtype=np.float32)
    fn = lib().tfo_int4_gemv_kernel_order if mat.bits == 4 else lib().tfo_int8_gemv_kernel_order
    fn(_p(mat.packed), _p(mat.scales), _p(mat.biases), mat.sb_dtype, _p(x), _p(y16), _p(y32), mat.m, mat.n)
    return y16, y32


# ---------------------------------------------------------------------------
# router
# ---------------------------------------------------------------------------

def router_logits(mat: AffineMatrix, hidden_f16: np.ndarray, eff_scale_bf16: np.ndarray,
                  stride: int | None = None) -> np.ndarray:
    hidden = np.ascontiguousarray(hidden_f16, dtype=np.uint16)
    if hidden.ndim == 1:
        hidden = hidden[None, :]
    T = hidden.shape[0]
    stride = hidden.shape[1] if stride is None else stride
    D = mat.n
    out = np.empty((T, mat.m), dtype=np.float32)
    lib().tfo_router_logits(_p(mat.packed), _p(mat.scales), _p(mat.biases), _p(hidden), stride,
                            _p(np.ascontiguousarray(eff_scale_bf16, dtype=np.uint16)), _p(out), T, mat.m, D)
    return out


def router_logits_f64(mat: AffineMatrix, hidden_f16: np.ndarray, eff_scale_bf16: np.ndarray) -> np.ndarray:
    hidden = np.ascontiguousarray(hidden_f16, dtype=np.uint16)
    if hidden.ndim == 1:
        hidden = hidden[None, :]
    T = hidden.shape[0]
    out = np.empty((T, mat.m), dtype=np.float64)
    lib().tfo_router_logits_f64(_p(mat.packed), _p(mat.scales), _p(mat.biases), _p(hidden), hidden.shape[1],
                                _p(np.ascontiguousarray(eff_scale_bf16, dtype=np.uint16)), _p(out), T, mat.m, mat.n)
    return out


def router_select(logits: np.ndarray, per_expert_scale_bf16: np.ndarray, k: int):
    """(indices u32 [T,k], weights fp16 bits [T,k], weights f32 [T,k])."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    if logits.ndim == 1:
        logits = logits[None, :]
    T, E = logits.shape
    idx = np.empty((T, k), dtype=np.uint32)
    w16 = np.empty((T, k), dtype=np.uint16)
    w32 = np.empty((T, k), dtype=np.float32)
    lib().tfo_router_select(_p(logits), _p(np.ascontiguousarray(per_expert_scale_bf16, dtype=np.uint16)),
                            _p(idx), _p(w16), _p(w32), T, E, k)
    return idx, w16, w32


def router_select_sorted(logits: np.ndarray, expert_scale_f32: np.ndarray, k: int):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    idx = np.empty(k, dtype=np.uint32)
    w = np.empty(k, dtype=np.float32)
    lib().tfo_router_select_sorted(_p(logits), _p(np.ascontiguousarray(expert_scale_f32, dtype=np.float32)),
                                   _p(idx), _p(w), logits.shape[0], k)
    return idx, w


# ---------------------------------------------------------------------------
# expert blobs
# ---------------------------------------------------------------------------

def blob_layout(D: int, F: int, align: int = 16384):
    """Byte offsets of gate{W,S,B} | up{W,S,B} | down{W,S,B} inside one expert blob
    and the aligned stride (Sources/TurboFieldfareRepack/Core/Planning/RepackPlanner.swift:337-399)."""
    gw = F * D // 2
    gs = F * (D // 64) * 2
    dw = D * F // 2
    ds = D * (F // 64) * 2
    off = ExpertOffsets()
    cur = 0
    for name, size in (("gate_w", gw), ("gate_s", gs), ("gate_b", gs), ("up_w", gw), ("up_s", gs), ("up_b", gs),
                       ("down_w", dw), ("down_s", ds), ("down_b", ds)):
        setattr(off, name, cur)
        cur += size
    payload = cur
    stride = (payload + align - 1) // align * align
    return off, payload, stride


def pack_blob(gate: AffineMatrix, up: AffineMatrix, down: AffineMatrix, off: ExpertOffsets, stride: int) -> np.ndarray:
    blob = np.zeros(stride, dtype=np.uint8)
    for name, arr in (("gate_w", gate.packed), ("gate_s", gate.scales), ("gate_b", gate.biases),
                      ("up_w", up.packed), ("up_s", up.scales), ("up_b", up.biases),
                      ("down_w", down.packed), ("down_s", down.scales), ("down_b", down.biases)):
        raw = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
        o = getattr(off, name)
        blob[o:o + raw.size] = raw
    return blob


def moe_routed_decode(blobs: list[np.ndarray], off: ExpertOffsets, x_f16, w_f16, residual_f16, D, F, order=0):
    """Returns (y fp16 bits, y f32, acts fp16 bits [K,F])."""
    K = len(blobs)
    ptrs = (C.c_void_p * K)(*[b.ctypes.data for b in blobs])
    y16 = np.empty(D, dtype=np.uint16)
    y32 = np.empty(D, dtype=np.float32)
    acts = np.empty((K, F), dtype=np.uint16)
    lib().tfo_moe_routed_decode(ptrs, C.byref(off), _p(np.ascontiguousarray(x_f16, dtype=np.uint16)),
                                _p(np.ascontiguousarray(w_f16, dtype=np.uint16)),
                                _p(None if residual_f16 is None else np.ascontiguousarray(residual_f16, dtype=np.uint16)),
                                _p(y16), _p(y32), _p(acts), D, F, K, order)
    return y16, y32, acts


def shared_expert_int4(gate: AffineMatrix, up: AffineMatrix, down: AffineMatrix, x_f16, order=0):
    D, Fs = gate.n, gate.m
    y16 = np.empty(D, dtype=np.uint16)
    y32 = np.empty(D, dtype=np.float32)
    lib().tfo_shared_expert_int4(_p(gate.packed), _p(gate.scales), _p(gate.biases),
                                 _p(up.packed), _p(up.scales), _p(up.biases),
                                 _p(down.packed), _p(down.scales), _p(down.biases),
                                 _p(np.ascontiguousarray(x_f16, dtype=np.uint16)), _p(y16), _p(y32), D, Fs, order)
    return y16, y32


def moe_reduce_token_major(partials_f16, weights_f16, T, K, D):
    out = np.empty((T, D), dtype=np.uint16)
    lib().tfo_moe_reduce_token_major(_p(np.ascontiguousarray(partials_f16, dtype=np.uint16)),
                                     _p(np.ascontiguousarray(weights_f16, dtype=np.uint16)), _p(out), T, K, D)
    return out


# ---------------------------------------------------------------------------
# grouping
# ---------------------------------------------------------------------------

GROUPING_ERRORS = {
    1: "invalidQueryCount", 2: "invalidTopK", 3: "invalidNumExperts", 4: "invalidTileExpertCount",
    5: "pairCountMismatch", 6: "tokenOutOfRange", 7: "rankOutOfRange", 8: "expertOutOfRange",
    9: "duplicateTokenRank", 10: "expertSortKeyCountMismatch",
}


class GroupingError(ValueError):
    def __init__(self, code: int):
        super().__init__(GROUPING_ERRORS.get(code, str(code)))
        self.code = code
        self.case = GROUPING_ERRORS.get(code)


def make_token_expert_pairs(indices: np.ndarray, weights_f16: np.ndarray, query_count: int, top_k: int) -> np.ndarray:
    out = np.zeros(query_count * top_k, dtype=PAIR_DTYPE)
    lib().tfo_make_token_expert_pairs(_p(np.ascontiguousarray(indices, dtype=np.uint32)),
                                      _p(np.ascontiguousarray(weights_f16, dtype=np.uint16)), query_count, top_k, _p(out))
    return out


@dataclass
class GroupedRoutes:
    sorted_pairs: np.ndarray
    per_expert_offsets: np.ndarray
    per_expert_counts: np.ndarray
    groups: np.ndarray
    tiles: np.ndarray


def group_pairs(pairs: np.ndarray, query_count: int, top_k: int, num_experts: int,
                tile_expert_count: int = 16, expert_sort_keys=None) -> GroupedRoutes:
    pairs = np.ascontiguousarray(pairs, dtype=PAIR_DTYPE)
    n = pairs.shape[0]
    sorted_out = np.zeros(max(n, 1), dtype=PAIR_DTYPE)
    offs = np.zeros(max(num_experts, 1), dtype=np.uint32)
    cnts = np.zeros(max(num_experts, 1), dtype=np.uint32)
    groups = np.zeros(max(n, 1), dtype=GROUP_DTYPE)
    tiles = np.zeros(max(n, 1), dtype=TILE_DTYPE)
    ng, nt = C.c_int(0), C.c_int(0)
    keys = None if expert_sort_keys is None else np.ascontiguousarray(expert_sort_keys, dtype=np.uint64)
    rc = lib().tfo_group_pairs(_p(pairs), n, query_count, top_k, num_experts, tile_expert_count,
                               _p(keys), 0 if keys is None else keys.shape[0],
                               _p(sorted_out), _p(offs), _p(cnts), _p(groups), C.byref(ng), _p(tiles), C.byref(nt))
    if rc != 0:
        raise GroupingError(rc)
    return GroupedRoutes(sorted_out[:n], offs[:num_experts], cnts[:num_experts], groups[:ng.value], tiles[:nt.value])


def grouped_moe_pairs(pool: np.ndarray, expert_stride: int, off: ExpertOffsets, hidden: np.ndarray,
                      act_dtype: int, pairs: np.ndarray, D: int, F: int, K: int, T: int) -> np.ndarray:
    """Per-pair partials [T, K, D] (16-bit patterns) with the prefill kernels' rounding points."""
    hidden = np.ascontiguousarray(hidden, dtype=np.uint16)
    pairs = np.ascontiguousarray(pairs, dtype=PAIR_DTYPE)
    out = np.zeros((T, K, D), dtype=np.uint16)
    lib().tfo_grouped_moe_pairs(_p(pool), expert_stride, C.byref(off), _p(hidden), hidden.shape[1], act_dtype,
                                _p(pairs), pairs.shape[0], _p(out), D, F, K)
    return out


def int4_qmm_ref(mat: AffineMatrix, X: np.ndarray, act_dtype: int = 0) -> np.ndarray:
    X = np.ascontiguousarray(X, dtype=np.uint16)
    T = X.shape[0]
    Y = np.empty((T, mat.m), dtype=np.float32)
    lib().tfo_int4_qmm_ref(_p(mat.packed), _p(mat.scales), _p(mat.biases), _p(X), act_dtype, _p(Y), T, mat.m, mat.n)
    return Y


# ---------------------------------------------------------------------------
# norms
# ---------------------------------------------------------------------------

def rmsnorm(x_f16: np.ndarray, weight_bf16, eps: float = 1e-6) -> np.ndarray:
    x = np.ascontiguousarray(x_f16, dtype=np.uint16)
    if x.ndim == 1:
        x = x[None, :]
    T, D = x.shape
    out = np.empty_like(x)
    w = None if weight_bf16 is None else np.ascontiguousarray(weight_bf16, dtype=np.uint16)
    lib().tfo_rmsnorm(_p(x), _p(w), _p(out), T, D, D, eps)
    return out


def layer_tail(h2_f16, h1_f16, hidden_f16, w_postffn2_bf16, w_postffn_bf16, eps=1e-6, layer_scalar=1.0):
    h2 = np.ascontiguousarray(h2_f16, dtype=np.uint16).reshape(-1, np.shape(h2_f16)[-1])
    T, D = h2.shape
    hid = np.array(hidden_f16, dtype=np.uint16, copy=True).reshape(T, D)
    lib().tfo_layer_tail(_p(h2), _p(np.ascontiguousarray(h1_f16, dtype=np.uint16).reshape(T, D)), _p(hid),
                         _p(np.ascontiguousarray(w_postffn2_bf16, dtype=np.uint16)),
                         _p(np.ascontiguousarray(w_postffn_bf16, dtype=np.uint16)), T, D, D, eps, layer_scalar)
    return hid


def post_attn_setup(hidden_f16, attn_f16, w_post_attn_bf16, w_pre_ffn_bf16, w_pre_ffn2_bf16, eps: float = 1e-6):
    """The primitive chain the reference's test compares its fused kernel with
    (Tests/TurboFieldfare/Core/Kernels/Fusions/FusedPostAttentionSetupTests.swift:52-101): attn = rms(attn) * w_post;
    hidden = half(hidden + attn); dense = rms(hidden) * w_pre; routed = rms(hidden) * w_pre2; router = rms(hidden).
    Returns (hidden, dense, routed, router) as fp16 bits [T, D]."""
    a = rmsnorm(attn_f16, w_post_attn_bf16, eps)
    h = np.ascontiguousarray(hidden_f16, dtype=np.uint16).reshape(a.shape)
    hidden = f32_to_f16((f16_to_f32(h) + f16_to_f32(a)).astype(np.float32))
    return (hidden, rmsnorm(hidden, w_pre_ffn_bf16, eps), rmsnorm(hidden, w_pre_ffn2_bf16, eps), rmsnorm(hidden, None, eps))


def lm_head_greedy(hidden_f16, norm_weight_bf16, mat: AffineMatrix, eps: float = 1e-6):
    """CPU reference of the greedy LM head (Tests/TurboFieldfare/Core/Kernels/Fusions/LMHeadChainInt4Tests.swift:10-41):
    RMSNorm rounded to fp16, dequantise-then-dot per row in fp32, first strict maximum (a NaN or -inf never wins;
    index 0 when nothing does). Returns (token, logits f32)."""
    normed = f16_to_f32(rmsnorm(hidden_f16, norm_weight_bf16, eps)).reshape(-1)
    logits = gemv_ref(mat, normed, acc="f32")
    best_v, best_i = -np.inf, 0
    finite = np.where(np.isnan(logits), -np.inf, logits)
    if finite.size and np.max(finite) > -np.inf:
        best_i = int(np.argmax(finite))          # first occurrence of the maximum = strict '>' scan
    return best_i, logits


# ---------------------------------------------------------------------------
# metrics (Tolerance/RelError.swift:7-16)
# ---------------------------------------------------------------------------

def rel_error(actual: np.ndarray, reference: np.ndarray) -> float:
    a = np.asarray(actual, dtype=np.float64).reshape(-1)
    r = np.asarray(reference, dtype=np.float64).reshape(-1)
    return float(np.max(np.abs(a - r)) / max(np.max(np.abs(r)), 1e-6))


def rel_l2(actual: np.ndarray, reference: np.ndarray) -> float:
    a = np.asarray(actual, dtype=np.float64).reshape(-1)
    r = np.asarray(reference, dtype=np.float64).reshape(-1)
    return float(np.linalg.norm(a - r) / max(np.linalg.norm(r), 1e-30))


def num_threads() -> int:
    return int(lib().tfo_num_threads())
