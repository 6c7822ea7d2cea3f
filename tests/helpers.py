"""Shared helpers of the tests (not part of the package)."""
import json
import os

import torch


def load_plain(model_dir):
    """config.json dictionary and {name: float32 tensor}, read with the safetensors library
    (not with the package's own reader)."""
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as f:
        raw = json.load(f)
    w = {k: v.float() for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}
    return raw, w


def random_tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
