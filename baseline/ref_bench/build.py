#!/usr/bin/env python3
"""Builds ``baseline/_ref/ref_bench``: tianyuxbear/zedinfer's NVIDIA path for Qwen2 (its transformer_forward,
PagedForwardContext, BlockPool, its CUDA kernels, cuBLASLt product and FlashInfer wrappers), compiled unmodified with
nvcc for sm_100a, plus the driver ``main.cpp`` of this folder.

    python baseline/ref_bench/build.py /path/to/zedinfer

The reference builds with xmake and git submodules; neither is here, so this script names the same sources and
flags by hand (xmake.lua, xmake/device/nvidia.lua: ``--nv-gpu=y --flashinfer=y``, ENABLE_NVIDIA_API, USE_FLASHINFER,
FLASHINFER_ENABLE_BF16, relocatable device code) and takes the headers its submodules would provide from what the
image has: FlashInfer's headers, its CUTLASS and its CCCL from the installed ``flashinfer`` package, nlohmann/json
from the cuDNN frontend's include folder, and a no-op stand-in for the plog logging headers
(tests/golden/ref_harness/shim).  No file of the reference is changed or copied.
"""
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(ROOT, "baseline", "_ref")

OPS = ("add", "argmax", "embedding", "kv_scatter", "linear", "rms_norm", "rope", "sample", "self_attention", "swiglu")


def site_packages():
    import site
    for sp in site.getsitepackages():
        if os.path.isdir(os.path.join(sp, "flashinfer", "data", "include")):
            return sp
    raise SystemExit("the flashinfer package (for its headers) is not installed")


def main():
    if len(sys.argv) != 2 or not os.path.isdir(sys.argv[1]):
        sys.exit("usage: build.py <checkout of tianyuxbear/zedinfer>")
    ref = os.path.abspath(sys.argv[1])
    sp = site_packages()
    fi = os.path.join(sp, "flashinfer", "data")
    nj = os.path.join(sp, "include", "cudnn_frontend", "thirdparty")
    if not os.path.isfile(os.path.join(nj, "nlohmann", "json.hpp")):
        raise SystemExit("nlohmann/json.hpp not found")
    shim = os.path.join(ROOT, "tests", "golden", "ref_harness", "shim")
    obj = os.path.join(OUT, "obj")
    os.makedirs(obj, exist_ok=True)
    inc = ["-I", shim, "-I", f"{ref}/include", "-I", nj,
           "-I", f"{fi}/cccl/libcudacxx/include", "-I", f"{fi}/cccl/cub", "-I", f"{fi}/cccl/thrust",
           "-I", f"{fi}/include", "-I", f"{fi}/cutlass/include"]
    defs = ["-DENABLE_NVIDIA_API", "-DUSE_FLASHINFER", "-DFLASHINFER_ENABLE_BF16"]
    cu = [f"{ref}/src/backend/device/nvidia/nvidia_runtime_api.cu"]
    for op in OPS:
        cu += [f for f in glob.glob(f"{ref}/src/backend/ops/{op}/nvidia/*.cu")]
    cpp = [f"{ref}/src/frontend/models/{n}.cpp" for n in ("transformer_forward", "paged_forward_context", "qwen2",
                                                          "decode_scratch")]
    cpp += [f"{ref}/src/zedinfer/batch_context.cpp", f"{ref}/src/backend/kvcache/block_pool.cpp",
            f"{ref}/src/backend/tensor/tensor.cpp", f"{ref}/src/backend/device/runtime_api.cpp",
            f"{ref}/src/backend/device/cpu/cpu_runtime_api.cpp", f"{ref}/src/backend/ops/rearrange/op.cpp",
            f"{ref}/src/utils/types.cpp", f"{ref}/src/frontend/sampler/sampler.cpp",
            os.path.join(HERE, "main.cpp"), os.path.join(HERE, "stubs.cpp")]
    cpp += glob.glob(f"{ref}/src/backend/core/*/*.cpp") + glob.glob(f"{ref}/src/backend/ops/rearrange/cpu/*.cpp")
    for op in OPS:
        cpp.append(f"{ref}/src/backend/ops/{op}/op.cpp")
        cpp += [f for f in glob.glob(f"{ref}/src/backend/ops/{op}/cpu/*.cpp") if "onednn" not in f]
    cpp = [f for f in cpp if os.path.isfile(f)]

    def compile_one(src):
        name = src.replace(ref, "ref").replace(ROOT, "own").strip("/").replace("/", "_")
        o = os.path.join(obj, name + ".o")
        if os.path.isfile(o) and os.path.getmtime(o) > os.path.getmtime(src):
            return o
        if src.endswith(".cu"):
            cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-rdc=true",
                   "-Xcompiler=-fPIC", "--expt-relaxed-constexpr", "--expt-extended-lambda"] + defs + inc + ["-c", src, "-o", o]
        else:
            cmd = ["g++", "-std=c++17", "-O2", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-Wno-unknown-pragmas"] + defs + inc + \
                  ["-I", "/usr/local/cuda/include", "-c", src, "-o", o]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout[-4000:] + r.stderr[-6000:] + "\n")
            raise SystemExit(f"failed: {src}")
        print("compiled", os.path.relpath(src, ref) if src.startswith(ref) else os.path.relpath(src, ROOT), flush=True)
        return o

    with ThreadPoolExecutor(max_workers=8) as pool:
        objects = list(pool.map(compile_one, cu + cpp))
    exe = os.path.join(OUT, "ref_bench")
    link = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler=-fopenmp", "-o", exe] + objects + \
           ["-lcublas", "-lcublasLt", "-Xlinker", "-rpath=/usr/local/cuda/lib64"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(" ".join(link[:8]) + " ...\n" + r.stdout[-4000:] + r.stderr[-8000:] + "\n")
        raise SystemExit("link failed")
    print("built", exe)


if __name__ == "__main__":
    main()
