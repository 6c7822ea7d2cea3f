"""Greedy generation through the entry point under drawn settings: model sizes, page size, pool size
(from "one request barely fits" to "all fit"), requests running at once, batch size, portion size,
token budget, overlapped steps on or off, 32-bit or bfloat16 - all drawn from a seed, so that a run
can be repeated by its number.  Small pools preempt and recompute.  Every generated token must be the
plain implementation's arg-max given the tokens before it (or lie within the precision's reach of
it), every request gets all its tokens, and no page is lost."""
import math
import random

import pytest

import plain_llama as plain
from helpers import load_plain, random_tokens

pytestmark = pytest.mark.gpu


def _draw(seed):
    rng = random.Random(seed)
    hd = rng.choice([16, 32, 48, 64, 64, 80, 128, 128])
    n_kv, grp = rng.choice([1, 2, 3, 4, 8]), rng.choice([1, 2, 3, 4, 4, 8])
    raw = {"architectures": ["LlamaForCausalLM"], "hidden_size": 8 * rng.randint(6, 40),
           "intermediate_size": 8 * rng.randint(6, 80), "num_hidden_layers": rng.randint(1, 3),
           "num_attention_heads": n_kv * grp, "num_key_value_heads": n_kv, "head_dim": hd,
           "vocab_size": rng.randint(100, 5000), "max_position_embeddings": 2048, "rms_norm_eps": 1e-5,
           "rope_theta": 10000.0, "rope_scaling": None, "tie_word_embeddings": False, "hidden_act": "silu"}
    page = rng.choice([8, 16, 16, 32])
    n_req = rng.randint(1, 12)
    lens = [rng.choice([rng.randint(1, 20), rng.randint(20, 120), rng.randint(120, 400)]) for _ in range(n_req)]
    news = [rng.randint(1, 40) for _ in range(n_req)]
    one = -(-max(l + n for l, n in zip(lens, news)) // page) + 1            # the longest request and a page
    every = sum(-(-(l + n) // page) for l, n in zip(lens, news))
    n_pages = rng.choice([one, one + rng.randint(0, 8), max(one, every // 2), every + 4])
    options = dict(block_size=page, num_cache_blocks=n_pages, max_sequences=rng.choice([1, 2, 4, 8, 16]),
                   max_batch_size=rng.choice([1, 2, 4, 8, 32]), prefill_chunk_size=rng.choice([8, 16, 24, 64, 512]),
                   max_num_batched_tokens=rng.choice([32, 64, 256, 2048]), overlap_steps=rng.random() < 0.7,
                   dtype=rng.choice(["float32", "bfloat16"]))
    return raw, lens, news, options


@pytest.mark.parametrize("seed", range(5000, 5024))
def test_drawn_engine_run_matches_plain(tmp_path, seed):
    from nanoinfer_b200 import Engine, SamplingParams
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.weights import write_random_model
    raw, lens, news, options = _draw(seed)
    folder = str(tmp_path / "m")
    s = math.sqrt(1.5 / raw["hidden_size"])                 # peaked attention (tiny_configs.sharp)
    write_random_model(folder, raw, seed + 1, slot_std={"q": s, "k": s})
    raw_read, w = load_plain(folder)
    prompts = [random_tokens(raw["vocab_size"], n, (seed + 1) * 100 + i) for i, n in enumerate(lens)]
    eng = Engine.from_model_dir(folder, **options)
    eng.stop_token_ids = ()
    ids = [eng.add_request(p, n, SamplingParams.greedy()) for p, n in zip(prompts, news)]
    eng.run()
    ops.check_device_errors()
    for rid, p, n in zip(ids, prompts, news):
        out = eng.get_request_result(rid)
        assert len(out) == n, f"{options}: {len(out)} tokens instead of {n}"
        logits = plain.forward(raw_read, w, list(p) + list(out))          # teacher-forced on the engine's own tokens
        for i, tok in enumerate(out):
            row = logits[len(p) - 1 + i]
            reach = 1e-4 * max(1.0, row.abs().max().item()) if options["dtype"] == "float32" else 0.05 * row.abs().max().item()
            assert (row.max() - row[tok]).item() <= reach, \
                f"{options}: prompt of {len(p)}, new token {i}: engine {tok}, plain {int(row.argmax())}"
    eng.runner.cache.check_consistency()
    assert eng.runner.cache.num_free_pages() == options["num_cache_blocks"]
