"""Weights: safetensors by name, dtypes kept, one error for everything wrong, random mode."""
import json
import os

import pytest
import torch

from tiny_configs import TINY_A, TINY_B
from nanoinfer_b200.config import config_from_dict, load_config
from nanoinfer_b200.weights import (SafetensorsError, WeightError, load_weights, random_tensors,
                                    tensor_plan, write_random_model, write_safetensors)
from nanoinfer_b200.weights import safetensors_io as sio


def test_random_model_round_trip_and_library_agreement(tmp_path):
    d = str(tmp_path / "m")
    write_random_model(d, TINY_B, seed=1)
    cfg = load_config(d)
    w = load_weights(d, cfg)
    assert set(w) == {p.name for p in tensor_plan(cfg)}
    assert all(t.dtype == torch.bfloat16 for t in w.values())
    assert torch.all(w["model.norm.weight"] == 1.0)
    emb = w["model.embed_tokens.weight"].float()
    assert abs(emb.std().item() - 0.02) < 2e-3 and abs(emb.mean().item()) < 1e-3
    # the safetensors library reads the same bytes
    from safetensors.torch import load_file
    lib = load_file(os.path.join(d, "model.safetensors"))
    assert set(lib) == set(w) and all(torch.equal(lib[k], w[k]) for k in w)
    # same seed, same values; another seed, other values; a tensor does not depend on the others
    again = dict(random_tensors(cfg, 1))
    assert all(torch.equal(again[k], w[k]) for k in w)
    other = dict(random_tensors(cfg, 2))
    assert not torch.equal(other["lm_head.weight"], w["lm_head.weight"])
    tied = dict(random_tensors(config_from_dict(dict(TINY_B, tie_word_embeddings=True)), 1))
    assert torch.equal(tied["model.embed_tokens.weight"], w["model.embed_tokens.weight"])


def test_stored_dtypes_are_kept(tmp_path):
    d = str(tmp_path / "m")
    cfg = config_from_dict(TINY_A)
    tensors = dict(random_tensors(cfg, 0))
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float() * 1.00001   # not a bf16 value
    tensors["model.layers.0.mlp.up_proj.weight"] = tensors["model.layers.0.mlp.up_proj.weight"].half()
    os.makedirs(d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(TINY_A, f)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors.items())
    w = load_weights(d, cfg)
    assert w["model.norm.weight"].dtype == torch.float32
    assert torch.equal(w["model.norm.weight"], tensors["model.norm.weight"])
    assert w["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16
    assert w["model.embed_tokens.weight"].dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = str(tmp_path / "m")
    cfg = config_from_dict(TINY_A)
    tensors = dict(random_tensors(cfg, 0))
    del tensors["model.layers.1.mlp.down_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(64, 64, dtype=torch.bfloat16)
    tensors["model.layers.7.extra.weight"] = torch.zeros(3, dtype=torch.bfloat16)
    os.makedirs(d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(TINY_A, f)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors.items())
    with pytest.raises(WeightError) as ei:
        load_weights(d, cfg)
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.down_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.7.extra.weight"]
    assert e.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (32, 64), (64, 64))]
    text = str(e)
    for s in ("missing (2)", "model.norm.weight", "unexpected (1)", "model.layers.7.extra.weight",
              "expected [32, 64] found [64, 64]"):
        assert s in text


def test_tied_model_may_store_lm_head_untied_must(tmp_path):
    for raw, has_head, ok in ((TINY_A, True, True), (TINY_B, False, False)):
        d = str(tmp_path / f"m{ok}")
        cfg = config_from_dict(raw)
        tensors = dict(random_tensors(cfg, 0))
        if has_head:
            tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
        else:
            tensors.pop("lm_head.weight")
        os.makedirs(d)
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(raw, f)
        write_safetensors(os.path.join(d, "model.safetensors"), tensors.items())
        if ok:
            assert "lm_head.weight" not in load_weights(d, cfg)
        else:
            with pytest.raises(WeightError, match="lm_head.weight"):
                load_weights(d, cfg)


def test_broken_files(tmp_path):
    d = str(tmp_path / "m")
    write_random_model(d, TINY_A, seed=0)
    cfg = load_config(d)
    path = os.path.join(d, "model.safetensors")
    data = open(path, "rb").read()
    with open(path, "wb") as f:           # truncated
        f.write(data[:len(data) // 2])
    with pytest.raises(WeightError, match="truncated|beyond the end"):
        load_weights(d, cfg)
    with open(path, "wb") as f:           # nonsense header length
        f.write(b"\xff" * 8 + data[8:64])
    with pytest.raises(WeightError, match="header length"):
        load_weights(d, cfg)
    os.remove(path)
    with pytest.raises(WeightError, match="no .safetensors"):
        load_weights(d, cfg)
    with pytest.raises(SafetensorsError, match="cannot be stored"):
        write_safetensors(path, [("x", torch.zeros(2, dtype=torch.uint8))])


def test_sharded_folder(tmp_path):
    d = str(tmp_path / "m")
    cfg = config_from_dict(TINY_A)
    tensors = list(random_tensors(cfg, 0))
    os.makedirs(d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(TINY_A, f)
    write_safetensors(os.path.join(d, "model-00001-of-00002.safetensors"), tensors[:7])
    write_safetensors(os.path.join(d, "model-00002-of-00002.safetensors"), tensors[7:])
    w = load_weights(d, cfg)
    assert all(torch.equal(w[n], t) for n, t in tensors)


def test_buffers_that_exporters_store_beside_the_weights_are_passed_over(tmp_path):
    """Older exports of the architecture carry model.layers.N.self_attn.rotary_emb.inv_freq: the
    architecture declares the pattern, the loader neither reads nor reports such tensors - while any
    other stray tensor is still an error."""
    d = str(tmp_path / "m")
    cfg = config_from_dict(TINY_A)
    tensors = dict(random_tensors(cfg, 0))
    extra = {f"model.layers.{i}.self_attn.rotary_emb.inv_freq": torch.ones(8) for i in range(2)}
    os.makedirs(d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(TINY_A, f)
    write_safetensors(os.path.join(d, "model.safetensors"), list({**tensors, **extra}.items()))
    w = load_weights(d, load_config(d))
    assert set(w) == set(tensors)
    write_safetensors(os.path.join(d, "model.safetensors"),
                      list({**tensors, **extra, "model.layers.0.self_attn.stray": torch.ones(3)}.items()))
    with pytest.raises(WeightError) as err:
        load_weights(d, load_config(d))
    assert err.value.unexpected == ["model.layers.0.self_attn.stray"]
