"""Makes tests/golden/*.npz: logits of the reference's own PyTorch Llama (tools/model.py of
the reference project) on tiny random models, for the test that anchors tests/plain_llama.py.

Run once by hand from the repository root, with the reference project's path:
    python tests/golden/make_golden.py /path/to/NanoInfer

tools/model.py rotates interleaved pairs, fixes theta at 10000 with no scaling
(tools/model.py:228) and ties the output projection.  So configuration A is used as it is
(with rope_pairing "interleaved"); for B the sin/cos buffers are overwritten with the llama3
table of src/op/kernels/cpu/rope_kernel.cpp:117-153, written out again below, and the output
projection is untied.  The weights are those of the package's random-weights mode
(seed 0 for A, 1 for B), copied by name.
"""
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

from tiny_configs import TINY_A, TINY_B  # noqa: E402
from nanoinfer_b200.config import config_from_dict  # noqa: E402
from nanoinfer_b200.weights import random_tensors  # noqa: E402


def llama3_table(hd, n_pos, theta, sc):
    """sin/cos [n_pos, hd/2] as src/op/kernels/cpu/rope_kernel.cpp:117-153 fills them."""
    f32 = np.float32
    freqs = np.empty(hd // 2, dtype=np.float32)
    for p in range(hd // 2):
        freq = f32(1.0) / f32(math.pow(f32(theta), f32(p * 2) / f32(hd)))
        if sc is not None:
            wavelen = f32(2.0) * f32(math.pi) / freq
            low_wl = f32(sc["original_max_position_embeddings"]) / f32(sc["low_freq_factor"])
            high_wl = f32(sc["original_max_position_embeddings"]) / f32(sc["high_freq_factor"])
            if wavelen >= low_wl:
                freq = freq / f32(sc["factor"])
            elif wavelen > high_wl:
                smooth = (f32(sc["original_max_position_embeddings"]) / wavelen - f32(sc["low_freq_factor"])) / \
                         (f32(sc["high_freq_factor"]) - f32(sc["low_freq_factor"]))
                freq = (f32(1.0) - smooth) * freq / f32(sc["factor"]) + smooth * freq
        freqs[p] = freq
    ang = np.arange(n_pos, dtype=np.float32)[:, None] * freqs[None, :]
    return torch.from_numpy(np.cos(ang)), torch.from_numpy(np.sin(ang))


def run(raw, seed, prompts, ref_root):
    sys.path.insert(0, os.path.join(ref_root, "tools"))
    from model import ModelArgs, Transformer
    raw = dict(raw, rope_pairing="interleaved")
    cfg = config_from_dict(raw)
    w = {n: t.float() for n, t in random_tensors(cfg, seed)}
    args = ModelArgs(dim=raw["hidden_size"], n_layers=raw["num_hidden_layers"],
                     n_heads=raw["num_attention_heads"], n_kv_heads=raw["num_key_value_heads"],
                     vocab_size=raw["vocab_size"], hidden_dim=raw["intermediate_size"],
                     norm_eps=raw["rms_norm_eps"], max_seq_len=raw["max_position_embeddings"])
    assert args.dim // args.n_heads == raw["head_dim"]
    m = Transformer(args).eval()
    if not raw["tie_word_embeddings"]:
        m.output.weight = torch.nn.Parameter(torch.empty_like(m.output.weight))
    sd = {"tok_embeddings.weight": w["model.embed_tokens.weight"], "norm.weight": w["model.norm.weight"]}
    sd["output.weight"] = w["model.embed_tokens.weight"] if raw["tie_word_embeddings"] else w["lm_head.weight"]
    for i in range(args.n_layers):
        p, q = f"model.layers.{i}", f"layers.{i}"
        sd[f"{q}.attention.wq.weight"] = w[f"{p}.self_attn.q_proj.weight"]
        sd[f"{q}.attention.wk.weight"] = w[f"{p}.self_attn.k_proj.weight"]
        sd[f"{q}.attention.wv.weight"] = w[f"{p}.self_attn.v_proj.weight"]
        sd[f"{q}.attention.wo.weight"] = w[f"{p}.self_attn.o_proj.weight"]
        sd[f"{q}.feed_forward.w1.weight"] = w[f"{p}.mlp.gate_proj.weight"]
        sd[f"{q}.feed_forward.w3.weight"] = w[f"{p}.mlp.up_proj.weight"]
        sd[f"{q}.feed_forward.w2.weight"] = w[f"{p}.mlp.down_proj.weight"]
        sd[f"{q}.attention_norm.weight"] = w[f"{p}.input_layernorm.weight"]
        sd[f"{q}.ffn_norm.weight"] = w[f"{p}.post_attention_layernorm.weight"]
    missing, unexpected = m.load_state_dict(sd, strict=False)
    assert not unexpected and all("freqs" in k for k in missing), (missing, unexpected)
    cos, sin = llama3_table(raw["head_dim"], raw["max_position_embeddings"], raw["rope_theta"],
                            raw["rope_scaling"])
    m.freqs_cos, m.freqs_sin = cos, sin
    out = {}
    with torch.no_grad():
        for i, prompt in enumerate(prompts):
            t = torch.tensor([prompt], dtype=torch.long)
            out[f"tokens_{i}"] = np.asarray(prompt, dtype=np.int32)
            out[f"logits_{i}"] = m(t, targets=t)[0].numpy().astype(np.float32)
    return out


def main():
    ref_root = sys.argv[1]
    g = torch.Generator().manual_seed(0)
    for name, raw, seed, lens in (("tiny_a", TINY_A, 0, (5, 33)), ("tiny_b", TINY_B, 1, (7, 90))):
        prompts = [torch.randint(0, raw["vocab_size"], (n,), generator=g).tolist() for n in lens]
        np.savez_compressed(os.path.join(HERE, f"{name}_reference_logits.npz"), **run(raw, seed, prompts, ref_root))
        print("wrote", name)


if __name__ == "__main__":
    main()
