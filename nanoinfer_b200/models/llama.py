"""The Llama architecture ("LlamaForCausalLM"): config.json keys and tensor names.

What the reference fixes in code for its Llama models (src/model/model.cpp:143-175:
eps 1e-5, rope theta, the llama3 scaling constants; head size = dim / heads,
src/model/model.cpp:179) is read here from config.json.  The layer structure is that
of src/model/llama.cpp:324-386: pre-norm blocks of grouped-query attention with
rotary positions and a SwiGLU feed-forward, RMSNorm everywhere, a final norm and an
output projection that may alias the embedding table.  Tensor names are the
safetensors names that the reference's exporter reads (tools/export_llama3.py:568-592).
"""
from __future__ import annotations

import math
from typing import Any, Dict, Tuple

from ..config.model_config import (ConfigError, FeedForwardSpec, LayerRun, LayerSpec, MixerSpec,
                                   ModelConfig, NormSpec, PositionSpec, RopeScaling, optional,
                                   require)
from ..config.registry import register_architecture

NAME = "LlamaForCausalLM"


def _rope_scaling(raw: Dict[str, Any]):
    rs = raw.get("rope_scaling")
    if rs is None:
        return None
    if not isinstance(rs, dict):
        raise ConfigError("config.json: 'rope_scaling' must be an object or null")
    rope_type = rs.get("rope_type", rs.get("type"))
    if rope_type in (None, "default"):
        return None
    if rope_type != "llama3":
        raise ConfigError(f"config.json: rope_scaling.rope_type '{rope_type}' is not supported "
                          f"(supported: llama3, default)")
    return RopeScaling(
        rope_type="llama3",
        factor=require(rs, "factor", float),
        low_freq_factor=require(rs, "low_freq_factor", float),
        high_freq_factor=require(rs, "high_freq_factor", float),
        original_max_position_embeddings=require(rs, "original_max_position_embeddings", int),
    )


def parse_config(raw: Dict[str, Any]) -> ModelConfig:
    hidden = require(raw, "hidden_size", int)
    inter = require(raw, "intermediate_size", int)
    n_layers = require(raw, "num_hidden_layers", int)
    n_heads = require(raw, "num_attention_heads", int)
    n_kv = optional(raw, "num_key_value_heads", int, n_heads)
    vocab = require(raw, "vocab_size", int)
    max_pos = require(raw, "max_position_embeddings", int)
    if n_heads <= 0 or n_kv <= 0 or n_layers <= 0 or inter <= 0:
        raise ConfigError("config.json: head counts, layer count and intermediate_size must be positive")
    if "head_dim" in raw and raw["head_dim"] is not None:
        head_dim = require(raw, "head_dim", int)
    else:
        if hidden % n_heads:
            raise ConfigError(f"config.json: hidden_size {hidden} is not a multiple of "
                              f"num_attention_heads {n_heads} and no head_dim is given")
        head_dim = hidden // n_heads
    if n_heads % n_kv:
        raise ConfigError(f"config.json: num_attention_heads {n_heads} is not a multiple of "
                          f"num_key_value_heads {n_kv}")
    if head_dim <= 0 or head_dim % 2:
        raise ConfigError(f"config.json: head_dim {head_dim} must be positive and even")
    act = optional(raw, "hidden_act", str, "silu")
    if act != "silu":
        raise ConfigError(f"config.json: hidden_act '{act}' is not supported (supported: silu)")
    for key in ("attention_bias", "mlp_bias"):
        if optional(raw, key, bool, False):
            raise ConfigError(f"config.json: {key}=true is not supported")
    eps = optional(raw, "rms_norm_eps", float, 1e-5)
    theta = optional(raw, "rope_theta", float, 10000.0)
    pairing = optional(raw, "rope_pairing", str, "half")
    if pairing not in ("half", "interleaved"):
        raise ConfigError(f"config.json: rope_pairing '{pairing}' must be 'half' or 'interleaved'")
    position = PositionSpec(kind="rope", theta=theta, rotary_dim=head_dim, pairing=pairing,
                            scaling=_rope_scaling(raw))
    mixer = MixerSpec(kind="attention", num_heads=n_heads, num_kv_heads=n_kv, head_dim=head_dim,
                      window=None, softmax_scale=1.0 / math.sqrt(head_dim), position=position)
    ffn = FeedForwardSpec(kind="swiglu", intermediate_size=inter)
    norm = NormSpec(kind="rmsnorm", eps=eps)
    layer = LayerSpec(mixer=mixer, feed_forward=ffn, mixer_norm=norm, ffn_norm=norm,
                      arrangement="pre_norm")
    eos = raw.get("eos_token_id")
    if eos is None:
        eos_ids: Tuple[int, ...] = ()
    elif isinstance(eos, int) and not isinstance(eos, bool):
        eos_ids = (eos,)
    elif isinstance(eos, list) and all(isinstance(e, int) for e in eos):
        eos_ids = tuple(eos)
    else:
        raise ConfigError("config.json: eos_token_id must be an integer or a list of integers")
    bos = raw.get("bos_token_id")
    if bos is not None and (not isinstance(bos, int) or isinstance(bos, bool)):
        raise ConfigError("config.json: bos_token_id must be an integer")
    return ModelConfig(
        architecture=NAME,
        hidden_size=hidden,
        vocab_size=vocab,
        max_position_embeddings=max_pos,
        layers=tuple(layer for _ in range(n_layers)),
        schedule=tuple(LayerRun(layer=i) for i in range(n_layers)),
        final_norm=norm,
        tie_word_embeddings=optional(raw, "tie_word_embeddings", bool, False),
        bos_token_id=bos,
        eos_token_ids=eos_ids,
        raw=tuple(sorted((k, repr(v)) for k, v in raw.items())),
    )


_MIXER = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj"}
_FFN = {"gate": "gate_proj", "up": "up_proj", "down": "down_proj"}


def tensor_name(scope: Tuple, slot: str) -> str:
    if scope == ("embedding",):
        return "model.embed_tokens.weight"
    if scope == ("lm_head",):
        return "lm_head.weight"
    if scope == ("final_norm",):
        return "model.norm.weight"
    if scope[0] == "layer":
        _, i, what = scope
        base = f"model.layers.{i}"
        if what == "mixer":
            return f"{base}.self_attn.{_MIXER[slot]}.weight"
        if what == "feed_forward":
            return f"{base}.mlp.{_FFN[slot]}.weight"
        if what == "mixer_norm":
            return f"{base}.input_layernorm.weight"
        if what == "ffn_norm":
            return f"{base}.post_attention_layernorm.weight"
    raise ConfigError(f"{NAME}: no tensor name for scope {scope} slot '{slot}'")


# Older exports of this architecture store each layer's rotary frequency buffer beside the weights.
register_architecture(NAME, parse_config, tensor_name, ignored_tensors=("*.rotary_emb.inv_freq",), replace=True)
