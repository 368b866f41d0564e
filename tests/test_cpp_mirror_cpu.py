"""The C++ host-side mirror (include/turbofieldfare.hpp) compiles against the C ABI, links to the library and reports
the missing device the way the Swift host would get MetalError.noDevice (no compute calls without a GPU)."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SRC = r'''
#include <cstdio>
#include <fstream>
#include <iterator>
#include <string>
#include <cuda_runtime_api.h>
#include "turbofieldfare.hpp"
namespace tf = turbofieldfare;
static std::string slurp(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    return std::string(std::istreambuf_iterator<char>(f), std::istreambuf_iterator<char>());
}
int main(int argc, char** argv) {
    std::printf("abi %d\n", tf_abi_version());
    if (argc > 1) {   // the frozen v1 documents of the reference parse on the host, no device involved
        const std::string dir = argv[1];
        try {
            tf::GTurboDirectory g(slurp(dir + "/manifest.json"), slurp(dir + "/layout.json"), slurp(dir + "/resident-index.bin"));
            const tf_gturbo_info i = g.info();
            std::printf("gturbo layers %u experts %u stride %llu second-expert offset %llu\n", i.num_layers, i.experts_per_layer,
                        (unsigned long long)i.expert_stride, (unsigned long long)g.expertOffset(0, 1));
            try { g.resident("missing.tensor"); return 5; }
            catch (const tf::Error& e) { std::printf("gturbo lookup status %d\n", e.status); }
        } catch (const tf::Error& e) {
            std::printf("gturbo failed %d: %s\n", e.status, e.what());
            return 6;
        }
    }
    int n = 0;
    const bool have_gpu = cudaGetDeviceCount(&n) == cudaSuccess && n > 0;
    try {
        tf::Context ctx(0);
        tf::DequantInt4GEMV gemv(ctx);
        tf::MoE moe(ctx);
        tf::PrefillRouter router(ctx);
        tf::PrefillGroupedRoutedMoE grouped(ctx);
        tf::MPPPrefillInt4QMM qmm(ctx);
        try {   // a Swift precondition (N % 64 == 0, DequantInt4GEMV.swift:57-62) becomes a thrown error, not a crash
            gemv.encode(nullptr, {&n, 0}, {&n, 0}, {&n, 0}, {&n, 0}, {&n, 0}, 4, 96);
            std::printf("no error\n");
            return 2;
        } catch (const tf::Error& e) {
            std::printf("status %d: %s\n", e.status, e.what());
        }
        std::printf("context ok\n");
    } catch (const tf::Error& e) {
        std::printf("status %d: %s\n", e.status, e.what());
        return have_gpu ? 3 : (e.status == TF_ERR_NO_DEVICE ? 0 : 4);
    }
    return 0;
}
'''


def test_cpp_mirror_compiles_links_and_reports_errors(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    from turbo_fieldfare_b200 import build as tf_build
    lib = tf_build.build(verbose=False)
    src = tmp_path / "mirror.cpp"
    src.write_text(SRC)
    exe = tmp_path / "mirror"
    cmd = [gxx, "-std=c++17", "-O1", "-I", str(ROOT / "include"), "-I", "/usr/local/cuda/include", str(src), "-o", str(exe),
           "-L", str(lib.parent), "-ltfcuda", f"-Wl,-rpath,{lib.parent}", "-L", "/usr/local/cuda/lib64", "-lcudart"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    run = subprocess.run([str(exe), str(ROOT / "tests" / "golden" / "gturbo_v1")], capture_output=True, text=True)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "abi 1" in run.stdout
    assert "gturbo layers 1 experts 2 stride 16384 second-expert offset 16384" in run.stdout
    assert "gturbo lookup status 205" in run.stdout
    assert "status" in run.stdout        # either the missing device or the rejected N
