"""CPU-side checks of the C-ABI library: it loads, exports every declared symbol,
keeps the pinned struct layouts, and its host-side routing metadata (no GPU work)
reproduces the reference's known-answer vectors and agrees with the oracle."""
import ctypes as C
import json
from pathlib import Path

import numpy as np
import pytest

from turbo_fieldfare_b200 import _capi
from turbo_fieldfare_b200.build import build

GOLDEN = Path(__file__).parent / "golden"


@pytest.fixture(scope="module")
def lib():
    build()
    return _capi.load()


def test_every_declared_symbol_is_exported_and_bound(lib):
    declared = _capi.declared_functions()
    assert len(declared) >= 15
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in _capi.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_capi.SIGNATURES) == set(declared)
    assert lib.tf_abi_version() == 1


def test_struct_layouts_match_the_reference_pins():
    assert C.sizeof(_capi.Pair) == 16
    assert [getattr(_capi.Pair, f).offset for f, _ in _capi.Pair._fields_] == [0, 4, 8, 12]
    assert C.sizeof(_capi.ExpertOffsets) == 36
    assert C.sizeof(_capi.Group) == 12 and C.sizeof(_capi.Tile) == 16
    assert C.sizeof(_capi.Projection) == 56


def test_no_cpu_fallback_without_a_device(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    handle = C.c_void_p()
    status = lib.tf_context_create(0, C.byref(handle))
    assert status == 8 and not handle.value          # TF_ERR_NO_DEVICE
    assert b"no CPU fallback" in lib.tf_last_error(None)


def _pairs(rows):
    from turbo_fieldfare_b200.kernels import PAIR_DTYPE
    a = np.zeros(len(rows), dtype=PAIR_DTYPE)
    for i, r in enumerate(rows):
        a[i] = tuple(r)
    return a


def test_host_grouping_known_answers(lib, oracle):
    from turbo_fieldfare_b200.kernels import PrefillMoEGrouping
    from test_oracle_pins import _check_grouping_case
    data = json.loads((GOLDEN / "grouping_vectors.json").read_text())
    for case in data["cases"]:
        _check_grouping_case(oracle, PrefillMoEGrouping.group_token_expert_pairs, case)


def test_host_grouping_errors(lib):
    from turbo_fieldfare_b200.kernels import PrefillMoEGrouping, PrefillMoEGroupingError
    data = json.loads((GOLDEN / "grouping_vectors.json").read_text())
    for err in data["errors"]:
        with pytest.raises(PrefillMoEGroupingError) as ei:
            PrefillMoEGrouping.group_token_expert_pairs(_pairs(err["pairs"]), err["query_count"], err["top_k"],
                                                        err["num_experts"], err["tile_expert_count"], err["sort_keys"])
        assert ei.value.case == err["case"]
    with pytest.raises(PrefillMoEGroupingError) as ei:
        PrefillMoEGrouping.group_token_expert_pairs(_pairs([[0, 0, 0, 1]]), 2, 1, 1, 1)
    assert ei.value.case == "pairCountMismatch"
    with pytest.raises(PrefillMoEGroupingError) as ei:
        PrefillMoEGrouping.group_token_expert_pairs(_pairs([[1, 0, 0, 1]]), 1, 1, 1, 1)
    assert ei.value.case == "tokenOutOfRange"
    with pytest.raises(PrefillMoEGroupingError) as ei:
        PrefillMoEGrouping.group_token_expert_pairs(_pairs([[0, 0, 3, 1]]), 1, 1, 1, 1)
    assert ei.value.case == "rankOutOfRange"
    assert PrefillMoEGrouping.group_token_expert_pairs(_pairs([]), 0, 8, 128, 16).groups.shape[0] == 0


@pytest.mark.parametrize("T,K,E,tile,keys", [(64, 8, 128, 16, False), (257, 8, 128, 8, True), (4096, 8, 128, 16, False),
                                             (5, 3, 7, 1, True)])
def test_host_grouping_matches_oracle_on_random_routes(lib, oracle, T, K, E, tile, keys):
    from turbo_fieldfare_b200.kernels import PrefillMoEGrouping, PrefillRouter
    rng = np.random.default_rng(T * 31 + K)
    idx = np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.uint32)
    w = rng.integers(0, 0x3C00, size=(T, K)).astype(np.uint16)
    pairs = PrefillRouter.make_token_expert_pairs(idx, w, T, K)
    assert pairs.tobytes() == oracle.make_token_expert_pairs(idx, w, T, K).tobytes()
    sort_keys = rng.integers(0, 5, size=E).astype(np.uint64) if keys else None
    shuffled = pairs[rng.permutation(len(pairs))]
    got = PrefillMoEGrouping.group_token_expert_pairs(shuffled, T, K, E, tile, sort_keys)
    ref = oracle.group_pairs(pairs, T, K, E, tile, sort_keys)
    assert got.sorted_pairs.tobytes() == ref.sorted_pairs.tobytes()
    assert np.array_equal(got.per_expert_offsets, ref.per_expert_offsets)
    assert np.array_equal(got.per_expert_counts, ref.per_expert_counts)
    assert got.groups.tobytes() == ref.groups.tobytes() and got.tiles.tobytes() == ref.tiles.tobytes()


def test_streamed_params_layout_is_the_reference_one():
    """PrefillGroupedRoutedMoETests+Layout.swift:7-28: 128 bytes, the pinned member offsets."""
    from turbo_fieldfare_b200._capi import StreamedParams as P
    assert C.sizeof(P) == 128
    want = {"pair_start": 0, "pair_count": 4, "d": 8, "routed_intermediate": 12, "top_k": 16, "hidden_stride_elements": 20,
            "live_expert_count": 24, "local_expert": 28, "gate_w_off": 92, "down_b_off": 124}
    for name, offset in want.items():
        assert getattr(P, name).offset == offset, name
    assert P.local_expert.offset + 15 * 4 == 88           # localExpert15
