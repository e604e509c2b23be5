"""Tiny configurations and helpers shared by the tests.

Two configurations of the architecture that differ in every size and option:
layers 2/3, hidden 64/96, heads 4/3, key/value heads 2/1, head size 16/32,
intermediate 176/256, vocabulary 256/384, theta 1e4/1e6, window 16/none, eps
1e-5/1e-6; a third has a head size that is not hidden/heads and a vocabulary that
is no multiple of 8; a fourth has a head size and window that the tensor-core
attention kernels take; a sixth is wide enough for the split-K products of decode."""
from __future__ import annotations

import atexit
import os
import tempfile

import numpy as np
import torch

TINY_A = {
    "architectures": ["MistralForCausalLM"], "model_type": "mistral",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "intermediate_size": 176, "vocab_size": 256,
    "rope_theta": 10000.0, "sliding_window": 16, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
TINY_B = {
    "architectures": ["MistralForCausalLM"], "model_type": "mistral",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3,
    "num_key_value_heads": 1, "intermediate_size": 256, "vocab_size": 384,
    "rope_theta": 1000000.0, "sliding_window": None, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
TINY_C = {
    "architectures": ["MistralForCausalLM"], "model_type": "mistral",
    "num_hidden_layers": 2, "hidden_size": 80, "num_attention_heads": 6,
    "num_key_value_heads": 3, "head_dim": 48, "intermediate_size": 200, "vocab_size": 331,
    "rope_theta": 50000.0, "sliding_window": 70, "rms_norm_eps": 3e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
TINY_D = {
    "architectures": ["MistralForCausalLM"], "model_type": "mistral",
    "num_hidden_layers": 2, "hidden_size": 128, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 320, "vocab_size": 512,
    "rope_theta": 10000.0, "sliding_window": 40, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
TINY_E = {   # a width and an intermediate size that are no multiples of 8, an odd vocabulary
    "architectures": ["MistralForCausalLM"], "model_type": "mistral",
    "num_hidden_layers": 2, "hidden_size": 84, "num_attention_heads": 3,
    "num_key_value_heads": 3, "head_dim": 32, "intermediate_size": 100, "vocab_size": 259,
    "rope_theta": 10000.0, "sliding_window": None, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
TINY_F = {   # wide enough that the few-token products split K: the folded norm and the rotation
             # inside the q/k/v product run (they need K >= 385), with a vocabulary and an
             # intermediate size that are no multiples of 128
    "architectures": ["MistralForCausalLM"], "model_type": "mistral",
    "num_hidden_layers": 2, "hidden_size": 512, "num_attention_heads": 8,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 1416, "vocab_size": 1000,
    "rope_theta": 100000.0, "sliding_window": 100, "rms_norm_eps": 2e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
# The layer sizes of Mistral 7B (hidden 4096, 32 heads over 8 key/value heads of 128, intermediate
# 14336, window 4096) with two layers and a vocabulary of 4096, so that the folder stays below 1 GB.
REAL_SIZES = {
    "architectures": ["MistralForCausalLM"], "model_type": "mistral",
    "num_hidden_layers": 2, "hidden_size": 4096, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 4096,
    "rope_theta": 10000.0, "sliding_window": 4096, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "F": TINY_F}


_made: list = []


def remove_model_dir(d: str) -> None:
    """Deletes a folder that `make_model_dir` made in a temporary place."""
    import shutil
    shutil.rmtree(d, ignore_errors=True)
    if d in _made:
        _made.remove(d)


@atexit.register
def _remove_all() -> None:
    for d in list(_made):
        remove_model_dir(d)


def make_model_dir(cfg: dict, seed: int, dtype=torch.bfloat16, where: str | None = None) -> str:
    """Writes a random model folder into a temporary place and returns it."""
    from torchless_rs_b200 import write_random_model
    from torchless_rs_b200.config import config_from_dict
    d = where
    if d is None:
        d = tempfile.mkdtemp(prefix="tl_model_")
        _made.append(d)          # removed when the interpreter exits, if not before
    # drawn on the GPU where there is one (the same bits as on the host, much faster)
    device = "cuda:0" if torch.cuda.is_available() and dtype != torch.float16 else "cpu"
    write_random_model(config_from_dict(cfg), d, seed, dtype, device)
    return d


def read_weights_numpy(model_dir: str) -> dict:
    """The folder's tensors as float32 numpy arrays, read with the `safetensors`
    package (not with the package under test)."""
    from safetensors import safe_open
    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k).to(torch.float32).numpy()
    return out


def random_tokens(rng: np.random.Generator, n: int, vocab: int) -> list:
    return [int(t) for t in rng.integers(0, vocab, size=n)]
