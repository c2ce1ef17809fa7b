"""Writes tests/golden/reference_anchor.json: outputs of kekzl/imp's own kernels on tiny inputs.

Needs a B200 and the reference's source tree.  The reference cannot be built as a project here (its
CMakeLists.txt wants CUDA >= 13.1 and fetches dependencies from the network), but its kernel files
compile one by one with nvcc 12.9.  This script compiles, UNMODIFIED and straight from the tree named
by IMP_REFERENCE_DIR, src/compute/{layernorm,rope,activation,embedding,sampling,attention}.cu with the
src/core and src/runtime files they need, links them with reference_anchor_driver.cu (this repository's
code: it calls the reference's public functions on small inputs, one launch per case), runs the result
once and stores its JSON.  tests/test_reference_anchor.py compares the plain implementation with those
numbers on every run, GPU or not.

    IMP_REFERENCE_DIR=/path/to/imp python tests/golden/make_reference_anchor.py [--out FILE]
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE_FILES = ["src/compute/layernorm.cu", "src/compute/rope.cu", "src/compute/activation.cu", "src/compute/embedding.cu",
                   "src/compute/sampling.cu", "src/compute/attention.cu", "src/core/tensor.cpp", "src/core/logging.cpp",
                   "src/runtime/pdl.cu"]


def build_and_run(reference_dir: str, workdir: str) -> dict:
    missing = [f for f in REFERENCE_FILES if not os.path.exists(os.path.join(reference_dir, f))]
    if missing:
        raise SystemExit(f"{reference_dir} is not the reference's tree: {missing[0]} is missing")
    exe = os.path.join(workdir, "reference_anchor")
    cmd = ["nvcc", "-arch=sm_100", "-O2", "-std=c++20", "--use_fast_math", "-DIMP_CUDA_13_1=0", "-Wno-deprecated-gpu-targets",
           "-I", os.path.join(reference_dir, "src"), "-I", os.path.join(reference_dir, "include"),
           os.path.join(HERE, "reference_anchor_driver.cu")] + [os.path.join(reference_dir, f) for f in REFERENCE_FILES] + ["-o", exe]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise SystemExit(f"the reference's files did not compile:\n{p.stderr[-4000:]}")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    if r.returncode != 0:
        raise SystemExit(f"the anchor program failed ({r.returncode}):\n{r.stderr[-2000:]}")
    return json.loads(r.stdout)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(HERE, "reference_anchor.json"))
    args = ap.parse_args()
    ref = os.environ.get("IMP_REFERENCE_DIR")
    if not ref:
        raise SystemExit("set IMP_REFERENCE_DIR to the reference's source tree")
    with tempfile.TemporaryDirectory() as d:
        data = build_and_run(ref, d)
    data["_how"] = ("outputs of kekzl/imp's unmodified kernels (nvcc 12.9, -arch=sm_100 --use_fast_math as the reference builds, "
                    "-DIMP_CUDA_13_1=0) on a B200; made by tests/golden/make_reference_anchor.py")
    with open(args.out, "w") as f:
        json.dump(data, f)
    print("wrote", args.out, {k: len(v) for k, v in data.items() if isinstance(v, list)})
    return 0


if __name__ == "__main__":
    sys.exit(main())
