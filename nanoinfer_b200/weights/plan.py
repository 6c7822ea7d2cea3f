"""The list of tensors a configuration needs: name, shape, initialisation rule.

Built from the parts' own ``weight_slots`` and the architecture's tensor naming, so
that the loader's check and the random-weights writer can never disagree with the
model that is assembled from the same configuration.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple

from ..config import registry
from ..config.model_config import ModelConfig


@dataclass(frozen=True)
class PlannedTensor:
    name: str
    shape: Tuple[int, ...]
    init: str
    scope: Tuple
    slot: str


def tensor_plan(config: ModelConfig) -> List[PlannedTensor]:
    arch = registry.architecture(config.architecture)
    d = config.hidden_size
    plan: List[PlannedTensor] = []

    def add(scope, slots):
        for slot, ws in slots.items():
            plan.append(PlannedTensor(arch.tensor_name(scope, slot), tuple(ws.shape), ws.init,
                                      scope, slot))

    emb = config.embedding_spec()
    add(("embedding",), registry.part("embedding", emb.kind).weight_slots(emb, d))
    for i, layer in enumerate(config.layers):
        add(("layer", i, "mixer_norm"),
            registry.part("norm", layer.mixer_norm.kind).weight_slots(layer.mixer_norm, d))
        add(("layer", i, "mixer"),
            registry.part("mixer", layer.mixer.kind).weight_slots(layer.mixer, d))
        add(("layer", i, "ffn_norm"),
            registry.part("norm", layer.ffn_norm.kind).weight_slots(layer.ffn_norm, d))
        add(("layer", i, "feed_forward"),
            registry.part("feed_forward", layer.feed_forward.kind).weight_slots(layer.feed_forward, d))
    add(("final_norm",),
        registry.part("norm", config.final_norm.kind).weight_slots(config.final_norm, d))
    head = config.head_spec()
    add(("lm_head",), registry.part("head", head.kind).weight_slots(head, d))
    names = [p.name for p in plan]
    if len(set(names)) != len(names):
        dup = sorted({n for n in names if names.count(n) > 1})
        raise ValueError(f"architecture '{config.architecture}' names tensors twice: {dup}")
    return plan
