"""`.gturbo` reader on CPU: the reference's frozen v1 fixtures, the rejection cases of its codec tests
(Tests/TurboFieldfareFormat/GTurboFormatCodecTests.swift:110-440) and a synthetic install on disk.
No GPU is needed: parsing is host code inside libtfcuda.so."""
import copy
import hashlib
import json
import struct
from pathlib import Path

import numpy as np
import pytest

from oracle import gturbo_writer as W
from turbo_fieldfare_b200.gturbo import GTurboDirectory, GTurboError

GOLDEN = Path(__file__).resolve().parent / "golden" / "gturbo_v1"
# Tests/TurboFieldfareFormatCompatibility/GTurboFormatCompatibilityTests.swift:59-63
DIGESTS = {
    "manifest.json": "f0c4d01ac7f1747416a0274dd26bb585e2e43ae294b02a8daf272e7129d46dce",
    "layout.json": "acf57a355128d1d8afb1d09b75dc1aa7fef98687871b1ff9f738dd511cb6e341",
    "resident-index.bin": "aa705246112c17d4b60422a2705bda53e96553f7ff96e09b00e6fbb5a4ffa594",
}
INVALID, OVERFLOW, TRUNCATED, IO, NOT_FOUND = 201, 202, 203, 204, 205
UNSUPPORTED, ALIGNMENT = 2, 4


def golden(name: str) -> bytes:
    return (GOLDEN / name).read_bytes()


def parse(manifest=None, layout=None, index=None) -> GTurboDirectory:
    def enc(doc, name):
        if doc is None:
            return golden(name)
        return doc if isinstance(doc, bytes) else json.dumps(doc).encode()
    return GTurboDirectory.parse(enc(manifest, "manifest.json"), enc(layout, "layout.json"),
                                 index if index is not None else golden("resident-index.bin"))


def rejected(status, **docs):
    with pytest.raises(GTurboError) as err:
        parse(**docs)
    assert err.value.status == status, err.value
    return err.value


def test_fixture_bytes_carry_the_digests_the_reference_pins():
    for name, digest in DIGESTS.items():
        assert hashlib.sha256(golden(name)).hexdigest() == digest


def test_writer_reproduces_the_frozen_fixtures_byte_for_byte():
    docs = W.frozen_fixture_documents()
    for name in DIGESTS:
        assert docs[name] == golden(name), name


def test_reader_on_the_frozen_fixtures():
    d = parse()
    i = d.info
    assert (i.version_major, i.version_minor) == (1, 0)
    assert (i.num_layers, i.experts_per_layer, i.top_k) == (1, 2, 1)
    assert (i.hidden_size, i.moe_intermediate_size, i.ffn_intermediate, i.shared_expert_bits) == (64, 32, 128, 4)
    assert (i.expert_stride, i.index_size, i.resident_size, i.entry_count) == (16384, 16384, 32, 1)
    # GTurboFormatCompatibilityTests.swift:41: layout.expert(layer: 0, expert: 1).offset == expertStride
    loc = d.expert(0, 1)
    assert (loc.file, loc.offset, loc.size, loc.physical_rank) == ("layer_00.bin", 16384, 16384, 1)
    assert d.resident_names() == ["language_model.model.embed_tokens.weight"]
    t = d.resident("language_model.model.embed_tokens.weight")
    assert t.dtype == "u32" and t.shape == (1, 1, 0, 0)
    # file offsets 16384 / 16400 / 16408 become payload-relative (Runtime/Inference/Model.swift:195-233)
    assert (t.offset, t.size, t.scale_offset, t.scale_size, t.bias_offset, t.bias_size) == (0, 16, 16, 8, 24, 8)
    with pytest.raises(GTurboError) as err:
        d.resident("language_model.model.norm.weight")
    assert err.value.status == NOT_FOUND
    with pytest.raises(GTurboError):
        d.expert(0, 2)
    with pytest.raises(GTurboError) as err:     # the fixture blob has no scale planes
        d.expert_offsets(0)
    assert err.value.status == INVALID
    d.close()


# ---- manifest ------------------------------------------------------------------------------------------
def manifest_doc():
    return json.loads(golden("manifest.json"))


def test_manifest_accepts_additive_minor_unknown_key_and_absent_optionals():
    m = manifest_doc()
    m["versionMinor"] = 7
    m["futureField"] = {"anything": [1, 2, 3]}
    parse(manifest=m).close()
    for key in ("sourceSnapshotHash", "quant", "bitWidthOverridesHonored"):
        m = manifest_doc()
        del m[key]
        d = parse(manifest=m)
        if key == "quant":
            assert d.info.shared_expert_bits == 0
        d.close()


@pytest.mark.parametrize("path", ["../escape.bin", "/absolute.bin", "a//b.bin", "a/./b.bin", "a/../b.bin", ""])
def test_manifest_rejects_unsafe_paths(path):
    m = manifest_doc()
    m["files"][path] = {"sha256": "0" * 64, "size": 1}
    rejected(INVALID, manifest=m)


def test_manifest_rejections():
    m = manifest_doc(); m["magic"] = "GTURBX"
    rejected(INVALID, manifest=m)
    m = manifest_doc(); m["versionMajor"] = 2
    rejected(UNSUPPORTED, manifest=m)
    m = manifest_doc(); m["flags"]["mystery"] = True
    rejected(INVALID, manifest=m)
    m = manifest_doc(); m["flags"]["turboQuantKV"] = True
    rejected(INVALID, manifest=m)
    m = manifest_doc(); m["expertStride"] = 16384 + 256
    rejected(ALIGNMENT, manifest=m)
    m = manifest_doc(); m["arch"]["numLayers"] = 2
    rejected(INVALID, manifest=m)
    m = manifest_doc(); m["files"]["MODEL_WEIGHTS.BIN"] = {"sha256": "0" * 64, "size": 1}     # case-insensitive collision
    rejected(INVALID, manifest=m)
    m = manifest_doc(); m["files"]["model_weights.bin"]["sha256"] = "xyz"
    rejected(INVALID, manifest=m)
    m = manifest_doc(); del m["files"]["packed_experts/layout.json"]
    rejected(IO, manifest=m)
    m = manifest_doc(); m["quant"]["router"]["weightBits"] = 4
    rejected(INVALID, manifest=m)
    m = manifest_doc(); m["quant"]["routedExpert"]["groupSize"] = 32
    rejected(INVALID, manifest=m)
    m = manifest_doc(); del m["expertStride"]
    rejected(INVALID, manifest=m)
    rejected(INVALID, manifest=b'{"magic" : "GTURBO", ')          # malformed JSON
    rejected(INVALID, manifest=golden("manifest.json") + b" x")   # trailing characters


# ---- layout --------------------------------------------------------------------------------------------
def layout_doc():
    return json.loads(golden("layout.json"))


def test_layout_identity_fallback_and_physical_ranks():
    lay = layout_doc()
    for e in lay["layers"][0]["experts"]:
        del e["expert"]                         # positional ids
    d = parse(layout=lay)
    assert d.expert(0, 1).offset == 16384
    d.close()
    lay = layout_doc()                          # logical 0 stored at rank 1 and vice versa
    e0, e1 = lay["layers"][0]["experts"]
    e0.update(physicalRank=1, offset=16384)
    e1.update(physicalRank=0, offset=0)
    d = parse(layout=lay)
    assert (d.expert(0, 0).offset, d.expert(0, 0).physical_rank) == (16384, 1)
    assert (d.expert(0, 1).offset, d.expert(0, 1).physical_rank) == (0, 0)
    d.close()


def test_layout_rejections():
    lay = layout_doc(); del lay["layers"][0]["experts"][1]["expert"]               # mixed explicit / positional
    rejected(INVALID, layout=lay)
    lay = layout_doc(); lay["layers"][0]["file"] = "nested/layer_00.bin"
    rejected(INVALID, layout=lay)
    for reserved in ("layout.json", "LAYOUT.JSON"):
        lay = layout_doc(); lay["layers"][0]["file"] = reserved
        rejected(INVALID, layout=lay)
    lay = layout_doc(); lay["layers"][0]["file"] = "layer_99.bin"                 # not in manifest.files
    rejected(INVALID, layout=lay)
    lay = layout_doc(); lay["layers"][0]["experts"][0]["tensors"]["gate"]["offset"] = 16384 - 16   # leaves the blob
    rejected(INVALID, layout=lay)
    lay = layout_doc(); lay["layers"].append(copy.deepcopy(lay["layers"][0])); lay["numLayers"] = 2
    rejected(INVALID, layout=lay)                                                 # duplicate layer id
    lay = layout_doc(); lay["layers"][0]["experts"][1]["expert"] = 0
    rejected(INVALID, layout=lay)                                                 # duplicate logical id
    lay = layout_doc(); lay["layers"][0]["experts"][0]["physicalRank"] = 1; lay["layers"][0]["experts"][0]["offset"] = 16384
    rejected(INVALID, layout=lay)                                                 # duplicate physical rank
    lay = layout_doc()
    lay["layers"][0]["experts"][0]["tensors"]["up"] = {"dtype": "U32", "offset": 16, "shape": [8, 8], "size": 32, "bits": 4}
    rejected(INVALID, layout=lay)                                                 # overlaps gate [0, 32)
    lay = layout_doc(); lay["layers"][0]["experts"][0]["tensors"]["gate"]["dtype"] = "FP8"
    rejected(INVALID, layout=lay)
    lay = layout_doc(); lay["layers"][0]["experts"][1]["offset"] = 32768          # not rank x stride
    rejected(INVALID, layout=lay)
    lay = layout_doc(); lay["expertStride"] = 32768                              # manifest says 16384
    rejected(INVALID, layout=lay)


# ---- resident index ------------------------------------------------------------------------------------
def index_entry(**kw):
    base = dict(name="a.weight", dtype=W.DTYPE_U32, fileOffset=16384, size=16, shape=[1, 1, 0, 0],
                scaleOffset=16400, scaleSize=8, biasOffset=16408, biasSize=8)
    base.update(kw)
    return base


def test_index_decodes_valid_regions():
    idx = W.resident_index([index_entry(), index_entry(name="b.weight", dtype=W.DTYPE_BF16, fileOffset=16416, size=32,
                                                       shape=[16, 0, 0, 0], scaleOffset=0, scaleSize=0, biasOffset=0,
                                                       biasSize=0)], 16384, 64)
    d = parse(index=idx)
    assert d.resident_names() == ["a.weight", "b.weight"]
    b = d.resident("b.weight")
    assert (b.dtype, b.offset, b.size, b.scale_size, b.bias_size, b.shape) == ("bf16", 32, 32, 0, 0, (16, 0, 0, 0))
    d.close()


def test_index_rejections():
    ok = bytearray(W.resident_index([index_entry()], 16384, 32))
    entry = 24
    # overlapping payload ranges
    rejected(INVALID, index=W.resident_index([index_entry(scaleOffset=16392)], 16384, 32))
    # name inside the entry table
    bad = bytearray(ok); struct.pack_into("<I", bad, entry, 30)
    rejected(INVALID, index=bytes(bad))
    # invalid UTF-8 name
    bad = bytearray(ok); bad[96] = 0xFF
    rejected(INVALID, index=bytes(bad))
    # nonzero reserved byte, unknown dtype
    bad = bytearray(ok); bad[entry + 7] = 1
    rejected(INVALID, index=bytes(bad))
    bad = bytearray(ok); bad[entry + 6] = 9
    rejected(INVALID, index=bytes(bad))
    # entry table larger than the index, and an entry count whose table size overflows 64 bits
    bad = bytearray(ok); struct.pack_into("<Q", bad, 16, 1 << 20)
    rejected(INVALID, index=bytes(bad))
    bad = bytearray(ok); struct.pack_into("<Q", bad, 16, 1 << 62)
    rejected(OVERFLOW, index=bytes(bad))
    # payload range outside the resident region
    rejected(INVALID, index=W.resident_index([index_entry(fileOffset=16384 + 64)], 16384, 32))
    rejected(INVALID, index=W.resident_index([index_entry(fileOffset=8192)], 16384, 32))
    # index region not a multiple of 16 KiB, larger than the data, header cut short
    bad = bytearray(ok); struct.pack_into("<Q", bad, 0, 16000)
    rejected(TRUNCATED, index=bytes(bad))
    bad = bytearray(ok); struct.pack_into("<Q", bad, 0, 32768)
    rejected(TRUNCATED, index=bytes(bad))
    rejected(TRUNCATED, index=bytes(ok[:20]))
    bad = bytearray(ok); struct.pack_into("<Q", bad, 0, 32 << 20)
    rejected(INVALID, index=bytes(bad))                                   # beyond the v1 metadata cap
    # empty primary payload, shapes, absent companion with an offset, duplicate names
    rejected(INVALID, index=W.resident_index([index_entry(size=0)], 16384, 32))
    rejected(INVALID, index=W.resident_index([index_entry(shape=[1, 0, 2, 0])], 16384, 32))
    rejected(INVALID, index=W.resident_index([index_entry(shape=[0, 0, 0, 0])], 16384, 32))
    rejected(INVALID, index=W.resident_index([index_entry(scaleSize=0)], 16384, 32))
    rejected(INVALID, index=W.resident_index([index_entry(), index_entry(fileOffset=16416, scaleOffset=0, scaleSize=0,
                                                                         biasOffset=0, biasSize=0)], 16384, 64))


# ---- a synthetic install on disk ------------------------------------------------------------------------
def small_install(root, rng, ranks=True):
    d, f, fs, experts, layers = 128, 64, 128, 4, 2
    table, payload = W.blob_tensor_table(d, f)
    blobs = [[rng.integers(0, 256, payload, dtype=np.uint8).tobytes() for _ in range(experts)] for _ in range(layers)]
    physical = [[3, 0, 2, 1], [1, 2, 3, 0]] if ranks else None
    resident = []
    for L in range(layers):
        p = f"language_model.model.layers.{L}"
        resident.append({"name": f"{p}.router.proj.weight", "dtype": W.DTYPE_U32, "shape": [experts, d // 4, 0, 0],
                         "weights": bytes(experts * d), "scales": bytes(experts * (d // 64) * 2),
                         "biases": bytes(experts * (d // 64) * 2)})
        resident.append({"name": f"{p}.router.scale", "dtype": W.DTYPE_BF16, "shape": [d, 0, 0, 0], "weights": bytes(2 * d)})
    meta = W.write_install(root, d=d, f=f, fs=fs, num_experts=experts, top_k=2, blobs=blobs, physical_ranks=physical,
                           resident=resident)
    return meta, blobs, physical


def test_open_a_directory_on_disk(tmp_path):
    meta, blobs, physical = small_install(tmp_path, np.random.default_rng(3))
    d = GTurboDirectory.open(tmp_path)
    i = d.info
    assert (i.num_layers, i.experts_per_layer, i.top_k, i.hidden_size, i.moe_intermediate_size) == (2, 4, 2, 128, 64)
    assert i.expert_stride == meta["stride"] and i.index_size == meta["index_size"] and i.resident_size == meta["resident_size"]
    off = d.expert_offsets(1)
    t = meta["table"]
    assert [off.gate_w_off, off.gate_s_off, off.gate_b_off, off.up_w_off, off.up_s_off, off.up_b_off,
            off.down_w_off, off.down_s_off, off.down_b_off] == [t[k]["offset"] for k in (
                "gate", "gate_scales", "gate_biases", "up", "up_scales", "up_biases", "down", "down_scales", "down_biases")]
    for L in range(2):
        for e in range(4):
            loc = d.expert(L, e)
            assert loc.file == f"layer_{L:02d}.bin" and loc.physical_rank == physical[L][e]
            assert loc.offset == physical[L][e] * meta["stride"]
            raw = (tmp_path / "packed_experts" / loc.file).read_bytes()[loc.offset:loc.offset + meta["payload"]]
            assert raw == blobs[L][e]
    r = d.resident("language_model.model.layers.1.router.proj.weight")
    assert r.size == 4 * 128 and r.scale_size == 4 * 2 * 2 and r.offset % 256 == 0
    d.close()


def test_open_reports_missing_and_inconsistent_files(tmp_path):
    with pytest.raises(GTurboError) as err:
        GTurboDirectory.open(tmp_path / "nowhere")
    assert err.value.status == IO
    small_install(tmp_path, np.random.default_rng(4), ranks=False)
    weights = tmp_path / "model_weights.bin"
    data = weights.read_bytes()
    weights.write_bytes(data[:-8])                        # shorter than the header says
    with pytest.raises(GTurboError) as err:
        GTurboDirectory.open(tmp_path)
    assert err.value.status == TRUNCATED
    weights.write_bytes(data + b"\0" * 8)                 # size differs from manifest.files
    with pytest.raises(GTurboError) as err:
        GTurboDirectory.open(tmp_path)
    assert err.value.status == INVALID
    weights.write_bytes(data)
    GTurboDirectory.open(tmp_path).close()
    (tmp_path / "packed_experts" / "layout.json").unlink()
    with pytest.raises(GTurboError) as err:
        GTurboDirectory.open(tmp_path)
    assert err.value.status == IO
