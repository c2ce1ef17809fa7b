"""Writes tests/golden/plain_tiny.json: logits of the plain implementation on two tiny random models.

These numbers pin the whole plain model (tests/plain/qwen3_plain.py) against accidental change; they
are not outputs of the reference, whose whole model cannot be built or run here (CUDA-only model
code, CUDA >= 13.1, network fetches).  What the reference's own kernels compute, part by part, is
stored in reference_anchor.json (see make_reference_anchor.py).  Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import os
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.path.insert(0, os.path.join(HERE, ".."))

from conftest import TINY  # noqa: E402
from imp_b200.config.registry import config_from_dict  # noqa: E402
from imp_b200.weights.random_init import write_model_folder  # noqa: E402
from plain.qwen3_plain import PlainModel  # noqa: E402


def main():
    out = {}
    for i, (name, (cd, std, _)) in enumerate(TINY.items()):
        with tempfile.TemporaryDirectory() as d:
            write_model_folder(d, config_from_dict(cd), seed=i + 1, std=std)
            m = PlainModel(d)
            g = torch.Generator().manual_seed(100 + i)
            ids = torch.randint(0, cd["vocab_size"], (40,), generator=g).tolist()
            lg = m.logits(ids)
            out[name] = {"ids": ids, "rows": [0, 1, 23, 24, 25, 39], "cols": [0, 1, 2, 3, cd["vocab_size"] - 1],
                         "logits": [[float(lg[r, c]) for c in [0, 1, 2, 3, cd["vocab_size"] - 1]]
                                    for r in [0, 1, 23, 24, 25, 39]],
                         "greedy": m.generate(ids[:5], 6)}
    with open(os.path.join(HERE, "plain_tiny.json"), "w") as f:
        json.dump(out, f)
    print("wrote", os.path.join(HERE, "plain_tiny.json"))


if __name__ == "__main__":
    main()
