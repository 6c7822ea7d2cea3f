"""Random-weights mode: write a model folder from a configuration and a seed.

Matrices are N(0, std) (std 0.02 by default, the init of the reference's training
model, tools/model.py:242-248); norm gains are 1.0.  Each tensor is drawn from a
generator seeded by (seed, tensor name), so a tensor's values do not depend on which
other tensors exist.  The folder holds config.json and model.safetensors, exactly what
the loader reads.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Iterator, Optional, Tuple

import torch

from ..config import registry
from .plan import tensor_plan
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensors(config, seed: int, std: float = 0.02, dtype: torch.dtype = torch.bfloat16,
                   slot_std: Optional[Dict[str, float]] = None) -> Iterator[Tuple[str, torch.Tensor]]:
    """``slot_std``: another standard deviation for the weights of some slots, by slot name (for
    instance {"q": 0.14, "k": 0.14} gives a model whose attention is peaked instead of nearly
    uniform; the values drawn are the same, scaled)."""
    slot_std = slot_std or {}
    for p in tensor_plan(config):
        if p.init == "ones":
            yield p.name, torch.ones(p.shape, dtype=dtype)
        elif p.init == "zeros":
            yield p.name, torch.zeros(p.shape, dtype=dtype)
        else:
            g = torch.Generator(device="cpu")
            g.manual_seed(_tensor_seed(seed, p.name))
            yield p.name, (torch.randn(p.shape, generator=g, dtype=torch.float32) * slot_std.get(p.slot, std)).to(dtype)


def write_random_model(model_dir: str, raw_config: Dict[str, Any], seed: int, std: float = 0.02,
                       dtype: torch.dtype = torch.bfloat16, slot_std: Optional[Dict[str, float]] = None) -> None:
    """Create ``model_dir`` with config.json (``raw_config`` as given) and model.safetensors."""
    config = registry.config_from_dict(raw_config)
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(raw_config, f, indent=1, sort_keys=True)
    write_safetensors(os.path.join(model_dir, "model.safetensors"),
                      random_tensors(config, seed, std, dtype, slot_std))
