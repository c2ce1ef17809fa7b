"""Shared fixtures: two tiny Qwen3 configurations that differ in every size and option,
model folders with random weights in temporary folders, and the `gpu` marker."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU (run with -m gpu)")


# A: 2 layers, hidden 64, 4 query / 2 kv heads of 16, tied head, theta 1e4, eps 1e-6, no window,
#    weights stored in float32.
TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "vocab_size": 256, "hidden_size": 64, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128,
    "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "tie_word_embeddings": True, "torch_dtype": "float32",
    "max_position_embeddings": 512,
}
# B: 3 layers, hidden 96, 6 query / 3 kv heads of 32 (6*32 != 96), inner 200, vocab 503, untied head,
#    theta 1e6, eps 1e-5, a 24-token window on layers 1 and 2, weights stored in bfloat16.
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "vocab_size": 503, "hidden_size": 96, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 32, "intermediate_size": 200,
    "rms_norm_eps": 1e-5, "rope_theta": 1000000.0, "tie_word_embeddings": False, "torch_dtype": "bfloat16",
    "use_sliding_window": True, "sliding_window": 24, "max_window_layers": 1, "max_position_embeddings": 1024,
}
# C: one query group (4 query heads on 1 kv head), head size 48 (a multiple of 16 that is no power of two),
#    width 80 and inner size 136 (no powers of two), vocab 131; layer_types mixes windows per layer.
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "vocab_size": 131, "hidden_size": 80, "num_hidden_layers": 4,
    "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 48, "intermediate_size": 136,
    "rms_norm_eps": 3e-6, "rope_theta": 50000.0, "tie_word_embeddings": True, "torch_dtype": "bfloat16",
    "sliding_window": 9, "layer_types": ["sliding_attention", "full_attention", "sliding_attention",
                                         "full_attention"], "max_position_embeddings": 768,
}
# D: head size 64 with two query heads per kv head, so that prompt portions of 64 tokens and more run on
#    the tensor-memory attention kernel (128-token tiles); a 100-token window on the first layer.
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"], "vocab_size": 211, "hidden_size": 112, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 152,
    "rms_norm_eps": 2e-6, "rope_theta": 300000.0, "tie_word_embeddings": False, "torch_dtype": "bfloat16",
    "sliding_window": 100, "layer_types": ["sliding_attention", "full_attention"], "max_position_embeddings": 1024,
}
# config, weight std, page size
TINY = {"A": (TINY_A, 0.05, 4), "B": (TINY_B, 0.08, 16), "C": (TINY_C, 0.06, 8), "D": (TINY_D, 0.06, 16)}


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name -> (folder, config dict, page size); folders are made once per session in a temporary place."""
    from imp_b200.config.registry import config_from_dict
    from imp_b200.weights.random_init import write_model_folder

    out = {}
    for i, (name, (cd, std, page)) in enumerate(TINY.items()):
        folder = str(tmp_path_factory.mktemp(f"tiny_{name}"))
        write_model_folder(folder, config_from_dict(cd), seed=i + 1, std=std)
        out[name] = (folder, cd, page)
    return out
