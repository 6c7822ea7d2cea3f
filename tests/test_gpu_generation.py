"""Generation through the Python entry point and the command line against the plain
implementation: greedy, temperature sampling, few pages (preemption), first tokens."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_llama as plain
import plain_sampling as ps
from helpers import load_plain, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# The engine's FP32 logits agree with the plain ones to rtol 1e-4 / atol 1e-5; divided by a
# temperature of 0.7 that moves a token's probability mass by up to about 2e-4 of itself.
LOGIT_ROUNDING = 2e-4


def _check_greedy(raw, w, prompt, generated, dtype):
    """Every generated token is the plain arg-max given the tokens before it - unless the
    plain top-2 logits are closer than the precision of the engine's dtype can tell apart."""
    seq = list(prompt)
    for i, tok in enumerate(generated):
        logits = plain.forward(raw, w, seq)[-1]
        top2 = torch.topk(logits, 2).values
        tol = 1e-4 if dtype == "float32" else 0.05 * logits.abs().max().item()
        if int(torch.argmax(logits)) != tok:
            assert (top2[0] - logits[tok]).item() <= tol, f"token {i}: engine {tok}, plain {int(torch.argmax(logits))}"
        seq.append(tok)


def _first_new_token(tokens, after=3):
    """Index of the first token from position ``after`` on that has not occurred before it."""
    return next(i for i in range(after, len(tokens)) if tokens[i] not in tokens[:i])


def _varied(tokens, least=6):
    """A continuation that keeps repeating one token (what a random model with a tied output
    produces: the last token's own embedding wins) would hide a corrupted cache, a skipped
    recompute or a wrong page.  The models of these tests must not be of that kind."""
    assert len(set(tokens)) >= least, f"degenerate plain continuation {tokens}: this model cannot show a fault"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key,page,lens,n_new", [("a", 16, [5, 17, 33], 16), ("b", 8, [1, 7, 40, 90, 130], 24),
                                                 ("ds", 16, [5, 17, 33, 70], 16), ("e", 16, [9, 40], 12)])
def test_greedy_generation_matches_plain(model_dirs, key, page, lens, n_new, dtype):
    from nanoinfer_b200 import Engine, SamplingParams
    raw, w = load_plain(model_dirs[key])
    raw = dict(raw, eos_token_id=None)
    prompts = [random_tokens(raw["vocab_size"], n, 50 + i) for i, n in enumerate(lens)]
    eng = Engine.from_model_dir(model_dirs[key], dtype=dtype, block_size=page, num_cache_blocks=64,
                                max_sequences=8, prefill_chunk_size=24)
    eng.stop_token_ids = ()
    outs = eng.generate(prompts, max_new_tokens=n_new, sampling_params=SamplingParams.greedy())
    for p, o in zip(prompts, outs):
        assert len(o) == n_new
        _check_greedy(raw, w, p, o, dtype)
        if dtype == "float32":
            assert o == plain.greedy_generate(raw, w, p, n_new)
    eng.runner.cache.check_consistency()
    assert eng.runner.cache.num_free_pages() == 64


def test_temperature_generation_follows_the_plain_stream(model_dirs):
    from nanoinfer_b200 import Engine, SamplingParams
    raw, w = load_plain(model_dirs["b"])
    prompts = [random_tokens(raw["vocab_size"], n, 70 + i) for i, n in enumerate([1, 7, 40, 90, 130])]
    eng = Engine.from_model_dir(model_dirs["b"], dtype="float32", block_size=8, num_cache_blocks=64,
                                max_sequences=8, prefill_chunk_size=24)
    eng.stop_token_ids = ()
    sp = SamplingParams(temperature=0.7, seed=1)
    outs = eng.generate(prompts, max_new_tokens=24, sampling_params=sp)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for i, tok in enumerate(o):
            want, acceptable, _ = ps.sample(plain.forward(raw, w, seq)[-1], 0.7, seed=1, index=i, rounding=LOGIT_ROUNDING)
            assert tok in acceptable, f"token {i}: engine {tok}, plain {want}"
            seq.append(tok)
    # the same requests one at a time give the same tokens: the stream does not depend on batching
    eng2 = Engine.from_model_dir(model_dirs["b"], dtype="float32", block_size=8, num_cache_blocks=64,
                                 max_sequences=1, prefill_chunk_size=512)
    eng2.stop_token_ids = ()
    assert eng2.generate(prompts, max_new_tokens=24, sampling_params=sp) == outs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key,page", [("ds", 16), ("bs", 8)])
def test_few_pages_force_preemption_and_tokens_stay_the_same(model_dirs, key, page, dtype):
    """So few pages that running requests are preempted and recomputed; the tokens are those of the
    plain implementation all the same (models whose continuations vary, see _varied)."""
    from nanoinfer_b200 import Engine, SamplingParams
    raw, w = load_plain(model_dirs[key])
    prompts = [random_tokens(raw["vocab_size"], n, 90 + i) for i, n in enumerate([30, 28, 25])]
    n_pages = 7 * 16 // page
    eng = Engine.from_model_dir(model_dirs[key], dtype=dtype, block_size=page, num_cache_blocks=n_pages,
                                max_sequences=4, prefill_chunk_size=16)
    eng.stop_token_ids = ()
    outs = eng.generate(prompts, max_new_tokens=40, sampling_params=SamplingParams.greedy())
    assert eng.get_scheduler_stats().num_preemptions >= 1
    for p, o in zip(prompts, outs):
        assert len(o) == 40
        want = plain.greedy_generate(raw, w, p, 40)
        _varied(want)
        if dtype == "float32":
            assert o == want
        else:
            _check_greedy(raw, w, p, o, dtype)
    eng.runner.cache.check_consistency()
    assert eng.runner.cache.num_free_pages() == n_pages


def test_sampled_generation_survives_preemption(model_dirs):
    """The second tiny configuration's own workload (prompts of 1, 7, 40, 90 and 130 tokens, 24 new
    tokens each at temperature 0.7 with seed 1, portions of 24, pages of 8) with so few pages that
    requests are preempted: after the recompute a request's draws go on with the index of its next
    token, so every token is still the plain sampler's."""
    from nanoinfer_b200 import Engine, SamplingParams
    raw, w = load_plain(model_dirs["b"])
    prompts = [random_tokens(raw["vocab_size"], n, 70 + i) for i, n in enumerate([1, 7, 40, 90, 130])]
    eng = Engine.from_model_dir(model_dirs["b"], dtype="float32", block_size=8, num_cache_blocks=38,
                                max_sequences=8, prefill_chunk_size=24)
    eng.stop_token_ids = ()
    sp = SamplingParams(temperature=0.7, seed=1)
    outs = eng.generate(prompts, max_new_tokens=24, sampling_params=sp)
    assert eng.get_scheduler_stats().num_preemptions >= 1
    assert all(eng.get_request(i).finish_reason == "length" for i in range(len(prompts)))
    for p, o in zip(prompts, outs):
        assert len(o) == 24
        _varied(o)
        seq = list(p)
        for i, tok in enumerate(o):
            want, acceptable, _ = ps.sample(plain.forward(raw, w, seq)[-1], 0.7, seed=1, index=i, rounding=LOGIT_ROUNDING)
            assert tok in acceptable, f"token {i}: engine {tok}, plain {want}"
            seq.append(tok)
    eng.runner.cache.check_consistency()
    assert eng.runner.cache.num_free_pages() == 38


def test_stop_token_from_config_ends_generation(model_dirs):
    from nanoinfer_b200 import Engine, SamplingParams
    raw, w = load_plain(model_dirs["ds"])
    prompt = random_tokens(raw["vocab_size"], 9, 3)
    free_run = plain.greedy_generate(raw, w, prompt, 12)
    _varied(free_run)
    first = _first_new_token(free_run)
    stop = free_run[first]
    eng = Engine.from_model_dir(model_dirs["ds"], dtype="float32")
    eng.stop_token_ids = (stop,)
    out = eng.generate([prompt], max_new_tokens=12, sampling_params=SamplingParams.greedy())[0]
    assert out == free_run[:first + 1]
    assert eng.get_request(0).finish_reason == "stop"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_overlapped_steps_change_no_token(model_dirs, dtype):
    """Launching a decode step from the ids still on the device gives the tokens of the engine that
    reads every step's ids first: greedy and sampled, with a stop token that is seen one step late."""
    from nanoinfer_b200 import Engine, SamplingParams
    raw, w = load_plain(model_dirs["ds"])
    prompts = [random_tokens(raw["vocab_size"], n, 20 + i) for i, n in enumerate([9, 3, 21])]
    params = [SamplingParams.greedy(), SamplingParams(temperature=0.8, top_k=20, seed=5), SamplingParams.greedy()]
    outs, feeds = [], []
    for overlap in (False, True):
        eng = Engine.from_model_dir(model_dirs["ds"], dtype=dtype, block_size=16, num_cache_blocks=32,
                                    max_sequences=4, overlap_steps=overlap)
        eng.stop_token_ids = ()
        free_run = eng.generate(prompts, max_new_tokens=20, sampling_params=params)
        _varied(free_run[0])
        stop = free_run[0][_first_new_token(free_run[0])]     # request 0 stops in mid-flight, not at its first token
        fed = [0]
        inner = eng.runner.step

        def counting(entries, device_tokens=None, inner=inner, fed=fed):
            fed[0] += device_tokens is not None
            return inner(entries, device_tokens=device_tokens) if device_tokens is not None else inner(entries)
        eng.runner.step = counting
        eng.stop_token_ids = (stop,)
        stopped = eng.generate(prompts, max_new_tokens=20, sampling_params=params)
        outs.append((free_run, stopped))
        feeds.append(fed[0])
        eng.runner.cache.check_consistency()
        assert eng.runner.cache.num_free_pages() == 32
    assert outs[0] == outs[1]
    assert feeds[0] == 0 and feeds[1] >= 5
    free_run, stopped = outs[1]
    at = _first_new_token(free_run[0])
    assert stopped[0] == free_run[0][:at + 1]
    # and against the plain implementation, not only engine against engine
    if dtype == "float32":
        assert free_run[0] == plain.greedy_generate(raw, w, prompts[0], 20)
        assert free_run[2] == plain.greedy_generate(raw, w, prompts[2], 20)
    else:
        _check_greedy(raw, w, prompts[0], free_run[0], dtype)


def test_command_line(model_dirs, tmp_path):
    raw, w = load_plain(model_dirs["ds"])
    prompt = random_tokens(raw["vocab_size"], 11, 4)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "nanoinfer"), "generate", "--model",
                           model_dirs["ds"], "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)),
                           "--max-new-tokens", "8", "--temperature", "0"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    rec = json.loads(proc.stdout.splitlines()[0])
    want = plain.greedy_generate(raw, w, prompt, 8)
    _varied(want, least=5)
    eos = raw.get("eos_token_id")
    stop = set([eos]) if isinstance(eos, int) else set(eos or [])
    cut = next((i + 1 for i, t in enumerate(want) if t in stop), len(want))
    assert rec["generated"] == want[:cut]
    # random-model writes a folder the loader accepts
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(raw))
    out = tmp_path / "m"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "nanoinfer"), "random-model", "--config",
                           str(cfg), "--seed", "0", "--out", str(out)], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    from safetensors.torch import load_file
    again = load_file(str(out / "model.safetensors"))
    from nanoinfer_b200.config import config_from_dict
    from nanoinfer_b200.weights import random_tensors
    fresh = dict(random_tensors(config_from_dict(raw), 0))
    assert set(again) == set(fresh) and all(torch.equal(again[k], fresh[k]) for k in fresh)
