"""Writes tests/golden/reference_safetensors_A.json: what the reference's own safetensors loader
(src/model/safetensors_loader.cpp, compiled here on the host) finds in the model.safetensors that
this repository's writer produces for tiny configuration A with seed 11 in bfloat16: every tensor's
dtype code (src/core/tensor.h:11-17), shape, byte size and a hash of its bytes.

    python tests/golden/make_safetensors_golden.py --reference DIR     # DIR: a checkout of Deyu-Kong/mini-infer
"""

import argparse
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import torch  # noqa: E402

import tiny  # noqa: E402

SEED = 11


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="a checkout of Deyu-Kong/mini-infer")
    args = ap.parse_args()
    ref = os.path.abspath(args.reference)
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "dump_reference_safetensors")
        subprocess.run(["nvcc", "-x", "cu", "-std=c++17", "-O1", "-I", os.path.join(ref, "src"),
                        "-I", os.path.join(ref, "third_party"), "-I", os.path.join(ref, "third_party", "nlohmann"),
                        os.path.join(HERE, "dump_reference_safetensors.cpp"),
                        os.path.join(ref, "src", "model", "safetensors_loader.cpp"),
                        os.path.join(ref, "src", "core", "tensor.cpp"), "-o", exe], check=True)
        folder = os.path.join(tmp, "model")
        tiny.make_folder(folder, tiny.CONFIGS["A"], seed=SEED, dtype=torch.bfloat16)
        out = subprocess.run([exe, os.path.join(folder, "model.safetensors")], check=True, capture_output=True,
                             text=True).stdout
        parsed = json.loads(out)
        with open(os.path.join(HERE, "reference_safetensors_A.json"), "w") as f:
            json.dump(parsed, f, indent=0, sort_keys=True)
            f.write("\n")
        print(len(parsed), "tensors")
    return 0


if __name__ == "__main__":
    sys.exit(main())
