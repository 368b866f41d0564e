"""Writer of `.gturbo` model directories. TEST INFRASTRUCTURE, like the rest of oracle/: the product only
reads the format (turbo_fieldfare_b200/csrc/gturbo.cpp); tests use this writer to build small installs and
to show, by reproducing the reference's frozen v1 fixtures byte for byte, that the format is understood.

Follows the reference's writers:
  * JSON documents: JSONSerialization with prettyPrinted + sortedKeys + withoutEscapingSlashes
    (Sources/TurboFieldfareFormat/GTurboPackedExpertsLayoutV1.swift:73-83, GTurboManifestV1.swift:159-170):
    two-space indent, `"key" : value`, one array element per line, keys in ascending order ignoring case,
    no final newline.
  * resident index: 24-byte header {indexSize, residentSize, entryCount}, 72-byte entries
    {u32 nameOffset, u16 nameLength, u8 dtype, u8 0, u64 fileOffset, u64 size, 4 x u32 shape,
     u64 scaleOffset, u64 scaleSize, u64 biasOffset, u64 biasSize}, the names, zero padding up to a multiple
    of 16 KiB (Sources/TurboFieldfareFormat/GTurboResidentIndexV1.swift:161-186, GTurboFormatV1.swift:7-10).
  * expert blobs: gate{W,S,B} | up{W,S,B} | down{W,S,B}, sub-tensor names `gate`, `gate_scales`, `gate_biases`, ...
    (Sources/TurboFieldfare/Runtime/Inference/ModelExpertIO.swift:21-40).
"""
from __future__ import annotations

import struct
from pathlib import Path

import numpy as np

ALIGNMENT = 16384
HEADER_BYTES, ENTRY_BYTES = 24, 72
DTYPE_U32, DTYPE_BF16, DTYPE_FP16, DTYPE_FP32 = 0, 1, 2, 3


def _number(v) -> str:
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, int):
        return str(v)
    if float(v).is_integer():
        return str(int(v))
    return repr(float(v))


def _string(s: str) -> str:
    out = ['"']
    for ch in s:
        if ch == '"':
            out.append('\\"')
        elif ch == "\\":
            out.append("\\\\")
        elif ch == "\n":
            out.append("\\n")
        elif ord(ch) < 0x20:
            out.append(f"\\u{ord(ch):04x}")
        else:
            out.append(ch)
    out.append('"')
    return "".join(out)


def foundation_json(value, indent: int = 0) -> str:
    """Pretty-printed, key-sorted JSON in Foundation's layout."""
    pad, inner = "  " * indent, "  " * (indent + 1)
    if isinstance(value, dict):
        rows = [f"{inner}{_string(k)} : {foundation_json(value[k], indent + 1)}" for k in sorted(value, key=lambda k: (k.lower(), k))]
        return "{\n" + ",\n".join(rows) + "\n" + pad + "}"
    if isinstance(value, (list, tuple)):
        rows = [f"{inner}{foundation_json(v, indent + 1)}" for v in value]
        return "[\n" + ",\n".join(rows) + "\n" + pad + "]"
    if isinstance(value, str):
        return _string(value)
    return _number(value)


def quant_slot(bits: int) -> dict:
    return {"biasType": "BF16", "groupSize": 64, "scaleType": "BF16", "scheme": "affine", "weightBits": bits}


def manifest_document(arch: dict, files: dict, experts_per_layer: int, num_layers: int, expert_stride: int,
                      model_id: str, source_snapshot_hash: str | None = None, bit_width_overrides: int | None = None,
                      shared_bits: int = 4) -> dict:
    doc = {
        "arch": arch,
        "expertsPerLayer": experts_per_layer,
        "expertStride": expert_stride,
        "files": {k: {"sha256": v[1], "size": v[0]} for k, v in files.items()},
        "flags": {"aneSharedExpert": False, "streamingPresent": True, "turboQuantKV": False},
        "magic": "GTURBO",
        "modelID": model_id,
        "numLayers": num_layers,
        "quant": {"attention": quant_slot(4), "embedding": quant_slot(4), "routedExpert": quant_slot(4),
                  "router": quant_slot(8), "sharedExpert": quant_slot(shared_bits)},
        "versionMajor": 1,
        "versionMinor": 0,
    }
    if source_snapshot_hash is not None:
        doc["sourceSnapshotHash"] = source_snapshot_hash
    if bit_width_overrides is not None:
        doc["bitWidthOverridesHonored"] = bit_width_overrides
    return doc


def layout_document(expert_stride: int, layers: list[dict]) -> dict:
    """layers: [{layer, file, experts: [{expert, physicalRank?, tensors: {name: {offset,size,dtype,shape,bits?}}}]}]."""
    out_layers = []
    for L in layers:
        experts = []
        for e in L["experts"]:
            physical = e.get("physicalRank", e["expert"])
            row = {"expert": e["expert"], "offset": physical * expert_stride, "size": expert_stride, "tensors": e["tensors"]}
            if "physicalRank" in e:
                row["physicalRank"] = e["physicalRank"]
            experts.append(row)
        out_layers.append({"experts": experts, "file": L["file"], "layer": L["layer"]})
    n_experts = len(layers[0]["experts"])
    return {"expertsPerLayer": n_experts, "expertStride": expert_stride, "layers": out_layers, "numLayers": len(layers)}


def resident_index(entries: list[dict], index_size: int, resident_size: int) -> bytes:
    """entries: [{name, dtype, fileOffset, size, shape(4), scaleOffset, scaleSize, biasOffset, biasSize}]."""
    table_end = HEADER_BYTES + ENTRY_BYTES * len(entries)
    names = b"".join(e["name"].encode() for e in entries)
    if table_end + len(names) > index_size or index_size % ALIGNMENT:
        raise ValueError("index does not fit index_size")
    out = bytearray(index_size)
    struct.pack_into("<QQQ", out, 0, index_size, resident_size, len(entries))
    cursor = table_end
    for k, e in enumerate(entries):
        name = e["name"].encode()
        shape = list(e["shape"]) + [0] * (4 - len(e["shape"]))
        struct.pack_into("<IHBBQQ4IQQQQ", out, HEADER_BYTES + k * ENTRY_BYTES, cursor, len(name), e["dtype"], 0,
                         e["fileOffset"], e["size"], *shape, e.get("scaleOffset", 0), e.get("scaleSize", 0),
                         e.get("biasOffset", 0), e.get("biasSize", 0))
        out[cursor:cursor + len(name)] = name
        cursor += len(name)
    return bytes(out)


# ---------------------------------------------------------------------------
# The reference's frozen fixture (Tests/TurboFieldfareFormatCompatibility/GTurboFormatCompatibilityTests.swift:66-165)
# ---------------------------------------------------------------------------
def frozen_fixture_documents() -> dict[str, bytes]:
    arch = {"attentionKEqV": True, "ffnIntermediate": 128, "finalLogitSoftcap": 30.0, "fullAttentionLayerMask": [0],
            "fullHeadDim": 32, "fullRopeTheta": 1_000_000.0, "headDim": 16, "hiddenActivation": "gelu_pytorch_tanh",
            "hiddenSize": 64, "moeIntermediateSize": 32, "numExperts": 2, "numFullKVHeads": 1, "numHeads": 4,
            "numKVHeads": 2, "numLayers": 1, "partialRotaryFactor": 0.25, "ropeTheta": 10_000.0, "slidingWindow": 128,
            "tieWordEmbeddings": True, "topKExperts": 1, "vocabSize": 1024}
    zero = "0" * 64
    stride = ALIGNMENT
    files = {"model_weights.bin": (ALIGNMENT + 32, zero), "packed_experts/layout.json": (1, zero),
             "packed_experts/layer_00.bin": (2 * stride, zero)}
    manifest = manifest_document(arch, files, 2, 1, stride, "fixture/model", "fixture-snapshot", 120)
    gate = {"bits": 4, "dtype": "U32", "offset": 0, "shape": [8, 8], "size": 32}
    layout = layout_document(stride, [{"layer": 0, "file": "layer_00.bin",
                                       "experts": [{"expert": 0, "tensors": {"gate": gate}},
                                                   {"expert": 1, "tensors": {"gate": gate}}]}])
    index = resident_index([{"name": "language_model.model.embed_tokens.weight", "dtype": DTYPE_U32,
                             "fileOffset": ALIGNMENT, "size": 16, "shape": [1, 1, 0, 0],
                             "scaleOffset": ALIGNMENT + 16, "scaleSize": 8, "biasOffset": ALIGNMENT + 24, "biasSize": 8}],
                           ALIGNMENT, 32)
    return {"manifest.json": foundation_json(manifest).encode(), "layout.json": foundation_json(layout).encode(),
            "resident-index.bin": index}


# ---------------------------------------------------------------------------
# Small synthetic installs
# ---------------------------------------------------------------------------
def _round_up(v: int, a: int) -> int:
    return (v + a - 1) // a * a


def blob_tensor_table(d: int, f: int) -> tuple[dict, int]:
    """Sub-tensor table of one routed-expert blob and its payload size."""
    table, cursor = {}, 0
    for role, rows, cols in (("gate", f, d), ("up", f, d), ("down", d, f)):
        w, sb = rows * cols // 2, rows * (cols // 64) * 2
        table[role] = {"bits": 4, "dtype": "U32", "offset": cursor, "shape": [rows, cols // 8], "size": w}
        cursor += w
        table[f"{role}_scales"] = {"dtype": "BF16", "offset": cursor, "shape": [rows, cols // 64], "size": sb}
        cursor += sb
        table[f"{role}_biases"] = {"dtype": "BF16", "offset": cursor, "shape": [rows, cols // 64], "size": sb}
        cursor += sb
    return table, cursor


def write_install(root: Path, *, d: int, f: int, fs: int, num_experts: int, top_k: int, blobs: list[list[bytes]],
                  physical_ranks: list[list[int]] | None, resident: list[dict], model_id: str = "synthetic/model") -> dict:
    """Writes a model directory.

    blobs[layer][logical expert] = payload bytes (gate|up|down planes); physical_ranks[layer][logical] = rank
    in the layer file (None: identity, and then the layout omits the field); resident = [{name, dtype, shape,
    weights: bytes, scales: bytes | None, biases: bytes | None}] in file order."""
    root = Path(root)
    (root / "packed_experts").mkdir(parents=True, exist_ok=True)
    layers = len(blobs)
    table, payload = blob_tensor_table(d, f)
    stride = _round_up(payload, ALIGNMENT)
    layout_layers, files = [], {}
    zero = "0" * 64
    for L in range(layers):
        name = f"layer_{L:02d}.bin"
        data = bytearray(num_experts * stride)
        experts = []
        for e in range(num_experts):
            rank = e if physical_ranks is None else physical_ranks[L][e]
            assert len(blobs[L][e]) == payload
            data[rank * stride:rank * stride + payload] = blobs[L][e]
            row = {"expert": e, "tensors": table}
            if physical_ranks is not None:
                row["physicalRank"] = rank
            experts.append(row)
        (root / "packed_experts" / name).write_bytes(bytes(data))
        files[f"packed_experts/{name}"] = (len(data), zero)
        layout_layers.append({"layer": L, "file": name, "experts": experts})
    layout_bytes = foundation_json(layout_document(stride, layout_layers)).encode()
    (root / "packed_experts" / "layout.json").write_bytes(layout_bytes)
    files["packed_experts/layout.json"] = (len(layout_bytes), zero)

    table_end = HEADER_BYTES + ENTRY_BYTES * len(resident)
    index_size = _round_up(table_end + sum(len(t["name"].encode()) for t in resident), ALIGNMENT)
    cursor, entries, payload_parts = index_size, [], []

    def place(data: bytes | None):
        nonlocal cursor
        if not data:
            return 0, 0
        pad = _round_up(cursor, 256) - cursor        # keep every plane 256-byte aligned in the payload
        payload_parts.append(b"\0" * pad)
        cursor += pad
        at = cursor
        payload_parts.append(data)
        cursor += len(data)
        return at, len(data)

    for t in resident:
        w_at, w_n = place(t["weights"])
        s_at, s_n = place(t.get("scales"))
        b_at, b_n = place(t.get("biases"))
        entries.append({"name": t["name"], "dtype": t["dtype"], "fileOffset": w_at, "size": w_n, "shape": t["shape"],
                        "scaleOffset": s_at, "scaleSize": s_n, "biasOffset": b_at, "biasSize": b_n})
    resident_size = cursor - index_size
    weights = resident_index(entries, index_size, resident_size) + b"".join(payload_parts)
    (root / "model_weights.bin").write_bytes(weights)
    files["model_weights.bin"] = (len(weights), zero)

    arch = {"attentionKEqV": True, "ffnIntermediate": fs, "finalLogitSoftcap": 30.0, "fullAttentionLayerMask": [0] * layers,
            "fullHeadDim": 32, "fullRopeTheta": 1_000_000.0, "headDim": 16, "hiddenActivation": "gelu_pytorch_tanh",
            "hiddenSize": d, "moeIntermediateSize": f, "numExperts": num_experts, "numFullKVHeads": 1, "numHeads": 4,
            "numKVHeads": 2, "numLayers": layers, "partialRotaryFactor": 0.25, "ropeTheta": 10_000.0,
            "slidingWindow": 128, "tieWordEmbeddings": True, "topKExperts": top_k, "vocabSize": 1024}
    manifest = manifest_document(arch, files, num_experts, layers, stride, model_id)
    (root / "manifest.json").write_bytes(foundation_json(manifest).encode())
    return {"stride": stride, "payload": payload, "table": table, "index_size": index_size, "resident_size": resident_size,
            "entries": entries}


def affine_planes(matrix) -> tuple[bytes, bytes, bytes]:
    """(codes, scales, biases) bytes of an oracle AffineMatrix."""
    return (np.ascontiguousarray(matrix.packed).tobytes(), np.ascontiguousarray(matrix.scales).tobytes(),
            np.ascontiguousarray(matrix.biases).tobytes())
