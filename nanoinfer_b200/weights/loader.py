"""Weights from a model folder, by tensor name, checked against the configuration.

Each tensor keeps the dtype it is stored in when that is bfloat16 or float32;
float16 becomes bfloat16, 64-bit integers become int32.  What a part computes in is
the part's decision.  Every problem of a folder is reported in ONE error: tensors
that are missing, tensors that nothing asks for, and tensors of a wrong shape.

The reference slices one memory-mapped file by position (src/model/llama.cpp:568-706)
and can only check counts afterwards (src/model/llama.cpp:727-764).
"""
from __future__ import annotations

from fnmatch import fnmatchcase
from typing import Dict, List

import torch

from ..config.model_config import ModelConfig
from . import safetensors_io as sio
from .plan import tensor_plan


class WeightError(ValueError):
    """The tensors of a model folder do not match its configuration."""

    def __init__(self, model_dir, missing, unexpected, wrong_shape, other=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.other = list(wrong_shape), list(other)
        lines = [f"weights in {model_dir} do not match config.json:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, found in self.wrong_shape:
            lines.append(f"  wrong shape: {name} expected {list(want)} found {list(found)}")
        for msg in self.other:
            lines.append(f"  {msg}")
        super().__init__("\n".join(lines))


def _stored_dtype(t: torch.Tensor) -> torch.Tensor:
    if t.dtype == torch.float16:
        return t.to(torch.bfloat16)
    if t.dtype == torch.int64:
        return t.to(torch.int32)
    return t


def check_tensors(model_dir: str, config: ModelConfig, found: Dict[str, tuple]) -> None:
    """Compare {name: shape} of a folder with the configuration's plan; raise WeightError."""
    plan = {p.name: p for p in tensor_plan(config)}
    missing = [n for n in plan if n not in found]
    from ..config import registry
    arch = registry.architecture(config.architecture)
    allowed_extra = set()
    if config.head_spec().tied:
        # a tied model may still store its output projection; it is not read
        allowed_extra.add(arch.tensor_name(("lm_head",), "weight"))
    unexpected = [n for n in found if n not in plan and n not in allowed_extra
                  and not any(fnmatchcase(n, pat) for pat in arch.ignored_tensors)]
    wrong = [(n, plan[n].shape, found[n]) for n in plan if n in found and tuple(found[n]) != plan[n].shape]
    if missing or unexpected or wrong:
        raise WeightError(model_dir, sorted(missing), sorted(unexpected), sorted(wrong))


def load_weights(model_dir: str, config: ModelConfig) -> Dict[str, torch.Tensor]:
    """Return {tensor name: host tensor} for every tensor the configuration needs."""
    files: List[str] = sio.list_files(model_dir)
    if not files:
        raise WeightError(model_dir, [], [], [], [f"no .safetensors file in {model_dir}"])
    entries: Dict[str, sio.TensorEntry] = {}
    problems = []
    for path in files:
        try:
            for name, e in sio.read_header(path).items():
                if name in entries:
                    problems.append(f"tensor '{name}' is stored in two files")
                entries[name] = e
        except sio.SafetensorsError as err:
            problems.append(str(err))
    if problems:
        raise WeightError(model_dir, [], [], [], problems)
    check_tensors(model_dir, config, {n: e.shape for n, e in entries.items()})
    out: Dict[str, torch.Tensor] = {}
    for p in tensor_plan(config):
        out[p.name] = _stored_dtype(sio.read_tensor(entries[p.name]))
    return out
