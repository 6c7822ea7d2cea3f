"""The tiny Llama configurations of the tests, as config.json dictionaries.

A and B differ in every size and option: layers, width, head counts and grouping, head
size, feed-forward width, vocabulary, rope theta and scaling, eps, tied or untied output.
C has sizes that are no power of two and a head size of 48.  D has the head size (64) and
grouping (4 query heads per key/value head) that the split-K decode kernel takes, and a width
that is not heads x head size.  E has heads of 128 in an odd group of three query heads per
key/value head (what the 3B size of the family has), an untied output and sizes that are no power
of two.  F is one thin layer under a vocabulary and a feed-forward wide enough for the routes that
only large output sizes take (the swapped-operand tensor-core product).

sharp(): standard deviations for the query and key projections that make the attention scores O(1)
(standard deviation about 1.5) instead of O(0.05), so that the softmax is peaked: a key that is
lost, or read from the wrong page, moves the logits by far more than bfloat16 rounding does.
(Not sharper than that: rounding errors of the scores grow with their size and pass through the
exponential, and the tolerances of these tests were fixed for scores of this order.)
"""
import math
TINY_A = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 64, "intermediate_size": 192, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "vocab_size": 256, "max_position_embeddings": 128, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "rope_scaling": None, "tie_word_embeddings": True,
    "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 96, "intermediate_size": 256, "num_hidden_layers": 3,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "vocab_size": 384, "max_position_embeddings": 512, "rms_norm_eps": 1e-6,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "tie_word_embeddings": False, "hidden_act": "silu", "eos_token_id": [2, 3],
}
TINY_C = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 120, "intermediate_size": 200, "num_hidden_layers": 2,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 48,
    "vocab_size": 1000, "max_position_embeddings": 2048, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 256},
    "tie_word_embeddings": True, "hidden_act": "silu",
}
TINY_D = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 160, "intermediate_size": 264, "num_hidden_layers": 2,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 64,
    "vocab_size": 520, "max_position_embeddings": 1024, "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 128},
    "tie_word_embeddings": True, "hidden_act": "silu",
}
TINY_E = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 192, "intermediate_size": 328, "num_hidden_layers": 2,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 128,
    "vocab_size": 777, "max_position_embeddings": 2048, "rms_norm_eps": 1e-6,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 512},
    "tie_word_embeddings": False, "hidden_act": "silu",
}
TINY_F = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 128, "intermediate_size": 6400, "num_hidden_layers": 1,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
    "vocab_size": 76000, "max_position_embeddings": 512, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "rope_scaling": None, "tie_word_embeddings": True, "hidden_act": "silu",
}
# D with an untied output: greedy continuations of a tied random model repeat the last token
TINY_D_UNTIED = dict(TINY_D, tie_word_embeddings=False)


def sharp(raw):
    """slot_std for write_random_model: scores q.k / sqrt(hd) with a standard deviation of about 1.5."""
    s = math.sqrt(1.5 / raw["hidden_size"])
    return {"q": s, "k": s}
