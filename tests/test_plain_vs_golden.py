"""The plain implementation against the committed outputs of the reference's own model code
(tests/golden/make_golden.py), and its own internal consistency."""
import os

import numpy as np
import pytest
import torch

import plain_llama as plain
from tiny_configs import TINY_A, TINY_B
from nanoinfer_b200.config import config_from_dict
from nanoinfer_b200.weights import random_tensors

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name,raw,seed", [("tiny_a", TINY_A, 0), ("tiny_b", TINY_B, 1)])
def test_plain_matches_reference_model(name, raw, seed):
    raw = dict(raw, rope_pairing="interleaved")
    w = {n: t.float() for n, t in random_tensors(config_from_dict(raw), seed)}
    gold = np.load(os.path.join(GOLDEN, f"{name}_reference_logits.npz"))
    for i in range(2):
        tokens = gold[f"tokens_{i}"].tolist()
        ours = plain.forward(raw, w, tokens).numpy()
        np.testing.assert_allclose(ours, gold[f"logits_{i}"], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("raw,seed", [(TINY_A, 0), (TINY_B, 1)])
def test_pairing_equivalence_under_row_permutation(raw, seed):
    """"half" pairing on safetensors-order q/k rows == "interleaved" on permuted rows."""
    w = {n: t.float() for n, t in random_tensors(config_from_dict(raw), seed)}
    tokens = torch.randint(0, raw["vocab_size"], (19,), generator=torch.Generator().manual_seed(3)).tolist()
    half = plain.forward(dict(raw, rope_pairing="half"), w, tokens)
    wp = dict(w)
    for i in range(raw["num_hidden_layers"]):
        p = f"model.layers.{i}.self_attn"
        wp[f"{p}.q_proj.weight"] = plain.permute_half_to_interleaved(w[f"{p}.q_proj.weight"], raw["num_attention_heads"])
        wp[f"{p}.k_proj.weight"] = plain.permute_half_to_interleaved(w[f"{p}.k_proj.weight"], raw["num_key_value_heads"])
    inter = plain.forward(dict(raw, rope_pairing="interleaved"), wp, tokens)
    torch.testing.assert_close(half, inter, rtol=1e-5, atol=1e-6)


def test_rope_inv_freq_matches_package_table():
    from nanoinfer_b200.config.model_config import RopeScaling
    from nanoinfer_b200.parts.position import rope_inverse_frequencies
    sc = TINY_B["rope_scaling"]
    ours = rope_inverse_frequencies(32, 500000.0, RopeScaling("llama3", sc["factor"], sc["low_freq_factor"],
                                                              sc["high_freq_factor"],
                                                              sc["original_max_position_embeddings"]))
    ref = plain.rope_inv_freq(32, 500000.0, sc).numpy()
    np.testing.assert_allclose(ours, ref, rtol=3e-7)
    # all three branches of the llama3 rule occur in this configuration
    base = plain.rope_inv_freq(32, 500000.0, None).numpy()
    ratio = ref / base
    assert (np.isclose(ratio, 1.0)).any() and (np.isclose(ratio, 1 / 32.0)).any()
    assert ((ratio > 1 / 32.0 + 1e-3) & (ratio < 1.0 - 1e-3)).any()


def test_attention_window_and_causality():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(9, 2, 16, generator=g) for _ in range(3))
    full = plain.attention(q, k, v, 0.25)
    win = plain.attention(q, k, v, 0.25, window=4)
    # with a window of 4 the first four queries see the same keys as without
    torch.testing.assert_close(full[:4], win[:4])
    assert not torch.allclose(full[6], win[6])
    # causality: changing a later key does not change an earlier output
    k2 = k.clone(); k2[7] += 1.0
    torch.testing.assert_close(plain.attention(q, k2, v, 0.25)[:7], full[:7])


def test_the_smoke_check_computes_what_the_plain_implementation_computes(tmp_path):
    """__graft_entry__.smoke() carries its own short restatement of the formulas; it must agree
    with the plain implementation of these tests."""
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import __graft_entry__ as entry
    from helpers import load_plain, random_tokens
    from nanoinfer_b200.weights import write_random_model
    raw = dict(entry.SMOKE_CONFIG, tie_word_embeddings=False)
    d = str(tmp_path / "m")
    write_random_model(d, raw, seed=0, slot_std={"q": 0.15, "k": 0.15})
    raw_read, w = load_plain(d)
    toks = random_tokens(raw["vocab_size"], 37, 1)
    torch.testing.assert_close(entry._plain_logits(raw, w, toks), plain.forward(raw_read, w, toks), rtol=1e-5, atol=1e-5)
