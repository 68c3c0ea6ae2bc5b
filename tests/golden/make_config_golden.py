"""Writes tests/golden/reference_config_<NAME>.json: what the reference's own configuration parser
(src/model/model_config.cpp, compiled here with plain g++; it is host-only) reads from the
config.json of each tiny configuration of tests/tiny.py.

    python tests/golden/make_config_golden.py --reference DIR     # DIR: a checkout of Deyu-Kong/mini-infer

The reference's model code itself (CUDA + cuBLAS, FP16, head sizes 64 and 128 only) cannot be built
or run on a CPU, so only this host-side parser is anchored by outputs of the reference; the plain
model of tests/plain_model.py rests on the reference's formulas.
"""

import argparse
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

import tiny  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="a checkout of Deyu-Kong/mini-infer")
    args = ap.parse_args()
    ref = os.path.abspath(args.reference)
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "dump_reference_config")
        subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ref, "src"),
                        "-I", os.path.join(ref, "third_party"), "-I", os.path.join(ref, "third_party", "nlohmann"),
                        os.path.join(HERE, "dump_reference_config.cpp"),
                        os.path.join(ref, "src", "model", "model_config.cpp"), "-o", exe], check=True)
        for name, cfg in sorted(tiny.CONFIGS.items()):
            path = os.path.join(tmp, f"config_{name}.json")
            with open(path, "w") as f:
                json.dump(cfg, f)
            out = subprocess.run([exe, path], check=True, capture_output=True, text=True).stdout
            parsed = json.loads(out)
            with open(os.path.join(HERE, f"reference_config_{name}.json"), "w") as f:
                json.dump(parsed, f, indent=1, sort_keys=True)
                f.write("\n")
            print(name, parsed)
    return 0


if __name__ == "__main__":
    sys.exit(main())
