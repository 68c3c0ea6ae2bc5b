"""Build the reference arm: the unmodified Deyu-Kong/mini-infer libraries plus the timing driver.

The reference is a CMake/C++ project (no setup.py, no pyproject.toml), so it is configured out
of tree into ``baseline/_ref/build`` with its own CMakeLists.txt and two of its cache variables
overridden (CMakeLists.txt:30-37): ``MINI_INFER_CUDA_ARCH=100`` and ``CUDAToolkit_ROOT``.
Nothing is written into the reference's source tree.  ``baseline/reference_bench.cpp`` is then
compiled against the reference's headers and linked with its static libraries into
``baseline/_ref/reference_bench``.

    python baseline/build_reference.py [--source /path/to/mini-infer]
"""

from __future__ import annotations

import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
BINARY = os.path.join(REF, "reference_bench")
LIBS = ["mini_infer_engine", "mini_infer_model", "mini_infer_layers", "mini_infer_kernels", "mini_infer_core"]


def build(source: str, cuda_root: str = "/usr/local/cuda", arch: str = "100") -> str:
    if not os.path.isfile(os.path.join(source, "CMakeLists.txt")):
        raise RuntimeError(f"no CMakeLists.txt under {source}")
    bdir = os.path.join(REF, "build")
    os.makedirs(bdir, exist_ok=True)
    nvcc = os.path.join(cuda_root, "bin", "nvcc")
    subprocess.run(["cmake", "-S", source, "-B", bdir, "-G", "Ninja", f"-DMINI_INFER_CUDA_ARCH={arch}",
                    f"-DCUDAToolkit_ROOT={cuda_root}", f"-DCMAKE_CUDA_COMPILER={nvcc}"], check=True)
    subprocess.run(["cmake", "--build", bdir, "--target", "mini_infer_engine", "-j", "16"], check=True)
    cmd = [nvcc, "-O2", "-std=c++17", "-x", "cu", f"-gencode=arch=compute_{arch},code=sm_{arch}",
           "-I", os.path.join(source, "src"), "-I", os.path.join(source, "third_party", "nlohmann"),
           os.path.join(HERE, "reference_bench.cpp"), "-o", BINARY, "-L", bdir]
    cmd += [f"-l{name}" for name in LIBS]
    cmd += ["-lcublas", "-lcuda"]
    subprocess.run(cmd, check=True)
    return BINARY


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--source", default=os.environ.get("MINI_INFER_REFERENCE", "/root/reference"))
    ap.add_argument("--cuda-root", default="/usr/local/cuda")
    args = ap.parse_args()
    try:
        print(build(args.source, args.cuda_root))
    except (subprocess.CalledProcessError, RuntimeError) as e:
        print(f"build_reference: {e}", file=sys.stderr)
        sys.exit(1)
