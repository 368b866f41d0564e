"""Regenerates tests/golden/gturbo_v1/ from the reference checkout.

The reference freezes three byte strings of its v1 model format as base64 files
(Tests/TurboFieldfareFormatCompatibility/Fixtures/v1/{manifest.json,layout.json,resident-index.bin}.base64)
and pins their SHA-256 digests in
Tests/TurboFieldfareFormatCompatibility/GTurboFormatCompatibilityTests.swift:59-63.
This script decodes them, checks the digests and stores the raw bytes as test fixtures.

    python tests/golden/make_gturbo_v1.py <path to the reference checkout>
"""
import base64
import hashlib
import sys
from pathlib import Path

DIGESTS = {
    "manifest.json": "f0c4d01ac7f1747416a0274dd26bb585e2e43ae294b02a8daf272e7129d46dce",
    "layout.json": "acf57a355128d1d8afb1d09b75dc1aa7fef98687871b1ff9f738dd511cb6e341",
    "resident-index.bin": "aa705246112c17d4b60422a2705bda53e96553f7ff96e09b00e6fbb5a4ffa594",
}


def main(reference: str) -> None:
    src = Path(reference) / "Tests" / "TurboFieldfareFormatCompatibility" / "Fixtures" / "v1"
    dst = Path(__file__).resolve().parent / "gturbo_v1"
    dst.mkdir(exist_ok=True)
    for name, digest in DIGESTS.items():
        raw = base64.b64decode((src / f"{name}.base64").read_text())
        got = hashlib.sha256(raw).hexdigest()
        if got != digest:
            raise SystemExit(f"{name}: sha256 {got} differs from the pinned {digest}")
        (dst / name).write_bytes(raw)
        print(f"{name}: {len(raw)} bytes, sha256 ok")


if __name__ == "__main__":
    main(sys.argv[1])
