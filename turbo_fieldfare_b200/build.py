"""In-tree build of ``libtfcuda.so`` (sm_100a only) with nvcc.

The shared library lands in ``turbo_fieldfare_b200/_lib/`` so that it travels
with the source tree; nothing is installed into site-packages and no JIT cache
is used. ``python -m turbo_fieldfare_b200.build`` rebuilds what is out of date.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "_lib"
OBJ_DIR = LIB_DIR / "obj"
LIB_PATH = LIB_DIR / "libtfcuda.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              "-Xptxas", "-warn-spills"]


def nvcc_path() -> str:
    for cand in (os.environ.get("TF_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set TF_NVCC")


def sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _headers_mtime() -> float:
    hs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((ROOT / "include").glob("*.h"))
    return max(h.stat().st_mtime for h in hs)


def _compile(src: Path, verbose: bool, extra: list[str]) -> Path:
    obj = OBJ_DIR / (src.name + ".o")
    newest = max(src.stat().st_mtime, _headers_mtime())
    if obj.exists() and obj.stat().st_mtime >= newest and not extra:
        return obj
    cmd = [nvcc_path(), *ARCH_FLAGS, *NVCC_FLAGS, *extra, "-I", str(ROOT / "include"), "-I", str(CSRC),
           "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}")
    if verbose and res.stdout.strip():
        print(f"[{src.name}]\n{res.stdout}")
    return obj


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> Path:
    """Compile every source under csrc/ for sm_100a and link libtfcuda.so."""
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    if force:
        for o in OBJ_DIR.glob("*.o"):
            o.unlink()
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose or ptxas_info, extra), srcs))
    if LIB_PATH.exists() and all(LIB_PATH.stat().st_mtime >= o.stat().st_mtime for o in objs):
        return LIB_PATH
    cmd = [nvcc_path(), *ARCH_FLAGS, "-shared", "-o", str(LIB_PATH), *[str(o) for o in objs]]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
