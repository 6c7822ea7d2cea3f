"""Typed model configuration.

A ``ModelConfig`` describes a decoder as data: a tuple of ``LayerSpec`` (each naming
its mixer, feed-forward, norms and their constants) and a ``schedule`` that lists, in
order, which layer runs and whose cache it reads.  Nothing here knows a concrete
architecture: an architecture's parser (registered in ``registry``) turns the keys of
its own ``config.json`` into these records.

The reference engine has no such file-level configuration: it reads seven integers
from a binary header (include/nanoinfer/model/config.h:13-21) and fixes every other
constant per model type in code (src/model/model.cpp:143-175).  Here every constant
comes from ``config.json``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, replace
from typing import Any, Dict, Optional, Tuple


class ConfigError(ValueError):
    """A configuration key is missing, has a wrong type or an unsupported value."""


@dataclass(frozen=True)
class RopeScaling:
    """Frequency rescaling rule of a rotary position encoding.

    ``rope_type == "llama3"`` is the piecewise rule of
    src/op/kernels/cpu/rope_kernel.cpp:117-139.
    """
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied by a mixer to its queries and keys.

    kind "rope": rotary; ``pairing`` "half" rotates (i, i + rotary_dim/2), which is
    what projection weights stored in the safetensors layout expect; "interleaved"
    rotates (2i, 2i+1), the reference kernels' convention
    (src/op/kernels/cpu/rope_kernel.cpp:68-93) for weights permuted by its exporter.
    kind "none": no encoding.
    """
    kind: str = "rope"
    theta: float = 10000.0
    rotary_dim: int = 0
    pairing: str = "half"
    scaling: Optional[RopeScaling] = None


@dataclass(frozen=True)
class NormSpec:
    kind: str = "rmsnorm"
    eps: float = 1e-5


@dataclass(frozen=True)
class MixerSpec:
    """Token mixer of a layer.  ``kind`` selects the registered part.

    For kind "attention": grouped-query attention over a paged key/value cache;
    ``window`` = number of most recent keys a query sees (itself included), or None
    for all keys; ``softmax_scale`` multiplies the scores (1/sqrt(head_dim) when the
    architecture does not say otherwise).  ``extra`` carries constants of mixers that
    are not attention.
    """
    kind: str = "attention"
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    softmax_scale: float = 0.0
    position: PositionSpec = field(default_factory=PositionSpec)
    extra: Tuple[Tuple[str, Any], ...] = ()

    def extra_dict(self) -> Dict[str, Any]:
        return dict(self.extra)


@dataclass(frozen=True)
class FeedForwardSpec:
    """Feed-forward of a layer.  kind "swiglu": down(silu(gate(x)) * up(x))."""
    kind: str = "swiglu"
    intermediate_size: int = 0
    extra: Tuple[Tuple[str, Any], ...] = ()

    def extra_dict(self) -> Dict[str, Any]:
        return dict(self.extra)


@dataclass(frozen=True)
class EmbeddingSpec:
    """How token ids become rows of the residual stream.  kind "table": row ``id`` of a
    [vocab, hidden] matrix (src/op/kernels/cuda/embedding_kernel.cu:7-31).  ``vocab_size`` 0 means
    the model's; ``extra`` carries constants of other kinds."""
    kind: str = "table"
    vocab_size: int = 0
    extra: Tuple[Tuple[str, Any], ...] = ()

    def extra_dict(self) -> Dict[str, Any]:
        return dict(self.extra)


@dataclass(frozen=True)
class HeadSpec:
    """How the residual stream's wanted rows become logits.  kind "linear": final norm, then a
    product with a [vocab, hidden] matrix (src/model/llama.cpp:381-389); ``tied``: that matrix is
    the embedding's table and the head stores none of its own."""
    kind: str = "linear"
    vocab_size: int = 0
    tied: bool = False
    extra: Tuple[Tuple[str, Any], ...] = ()

    def extra_dict(self) -> Dict[str, Any]:
        return dict(self.extra)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: how mixer, feed-forward and norms are arranged, and their specs.

    arrangement "pre_norm":  h += mixer(norm1(h)); h += ffn(norm2(h))
    (src/model/llama.cpp:324-379).
    """
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    mixer_norm: NormSpec
    ffn_norm: NormSpec
    arrangement: str = "pre_norm"


@dataclass(frozen=True)
class LayerRun:
    """One entry of the execution schedule.

    ``layer``: index into ``ModelConfig.layers`` (a layer may be named twice; its
    weights are shared, every run has a cache of its own).
    ``cache_of``: index of an earlier *run* whose cache this run reads instead of
    writing one of its own; None = own cache.
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelConfig:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position_embeddings: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[LayerRun, ...]
    final_norm: NormSpec
    tie_word_embeddings: bool = False
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    raw: Tuple[Tuple[str, Any], ...] = ()
    embedding: EmbeddingSpec = field(default_factory=EmbeddingSpec)
    head: HeadSpec = field(default_factory=HeadSpec)

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    def embedding_spec(self) -> EmbeddingSpec:
        """The embedding's spec with the model's vocabulary filled in."""
        return replace(self.embedding, vocab_size=self.embedding.vocab_size or self.vocab_size)

    def head_spec(self) -> HeadSpec:
        """The head's spec with the model's vocabulary and ``tie_word_embeddings`` filled in."""
        return replace(self.head, vocab_size=self.head.vocab_size or self.vocab_size,
                       tied=self.head.tied or self.tie_word_embeddings)

    def validate(self) -> None:
        if self.hidden_size <= 0 or self.vocab_size <= 0:
            raise ConfigError("hidden_size and vocab_size must be positive")
        if self.max_position_embeddings <= 0:
            raise ConfigError("max_position_embeddings must be positive")
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        if not self.schedule:
            raise ConfigError("the schedule is empty")
        for r, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ConfigError(f"schedule[{r}] names layer {run.layer}, "
                                  f"but there are {len(self.layers)} layers")
            if run.cache_of is not None:
                if not 0 <= run.cache_of < r:
                    raise ConfigError(f"schedule[{r}].cache_of={run.cache_of} must name an "
                                      f"earlier run")
                if self.schedule[run.cache_of].cache_of is not None:
                    raise ConfigError(f"schedule[{r}].cache_of={run.cache_of} names a run "
                                      f"that has no cache of its own")


def require(raw: Dict[str, Any], key: str, typ) -> Any:
    """Fetch a required key of the given type (int is accepted where float is asked)."""
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    return coerce(raw[key], key, typ)


def optional(raw: Dict[str, Any], key: str, typ, default: Any) -> Any:
    if key not in raw or raw[key] is None:
        return default
    return coerce(raw[key], key, typ)


def coerce(value: Any, key: str, typ) -> Any:
    if typ is float and isinstance(value, (int, float)) and not isinstance(value, bool):
        return float(value)
    if typ is int and isinstance(value, int) and not isinstance(value, bool):
        return value
    if typ is bool and isinstance(value, bool):
        return value
    if typ is str and isinstance(value, str):
        return value
    if typ is dict and isinstance(value, dict):
        return value
    raise ConfigError(f"config.json: key '{key}' should be {typ.__name__}, "
                      f"found {type(value).__name__} ({value!r})")


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir}")
    with open(path, "r", encoding="utf-8") as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return raw
