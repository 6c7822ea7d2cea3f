"""Replay on the GPU against the plain implementation: the same requests whole, with the
last 32 tokens one by one, in portions of changing size, and mixed with other requests so
that pages are used again - in 32-bit and in bfloat16."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import replay_util as ru
from helpers import load_plain, random_tokens

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# per configuration: page size and request lengths (up to max_position_embeddings)
SETUP = {
    "a": (16, [5, 17, 33, 64, 100, 128]),
    "b": (8, [1, 7, 40, 90, 130, 300, 47]),
    "c": (16, [3, 48, 250, 611, 97]),
    "d": (16, [2, 129, 700, 65, 310]),
    "ds": (16, [2, 129, 700, 65, 310]),       # D untied, peaked attention
    "e": (16, [3, 130, 515, 66, 300]),        # heads of 128 in groups of three, peaked attention
}
CUTS = {"whole": ru.whole, "tail": ru.tail_by_token, "ragged": ru.ragged, "mixed": ru.mixed}


def _requests(raw, lens, seed):
    return {f"r{i}": random_tokens(raw["vocab_size"], n, seed * 100 + i) for i, n in enumerate(lens)}


@pytest.fixture(scope="module")
def plain_cache():
    return {}


def _plain(plain_cache, key, model_dir):
    if key not in plain_cache:
        raw, w = load_plain(model_dir)
        page, lens = SETUP[key]
        reqs = _requests(raw, lens, seed=sum(map(ord, key)))
        plain_cache[key] = (raw, reqs, ru.plain_logits(raw, w, reqs))
    return plain_cache[key]


def _runner(model_dir, dtype, page, steps, max_requests=4):
    from nanoinfer_b200.config import load_config
    from nanoinfer_b200.engine import ModelRunner
    from nanoinfer_b200.weights import load_weights
    cfg = load_config(model_dir)
    # exactly as many pages as the trace needs at its fullest (requests rounded up to 64)
    num_pages = ru.max_live_tokens(steps, 64) // page
    return ModelRunner(cfg, load_weights(model_dir, cfg), dtype=dtype, page_size=page,
                       num_pages=num_pages, max_requests=max_requests)


class _Spy:
    """Counts the calls of one function of nanoinfer_b200.kernels.ops and keeps what ``note``
    extracts from each call's arguments; the function itself runs unchanged."""

    def __init__(self, monkeypatch, name, note):
        from nanoinfer_b200.kernels import ops
        self.seen = []
        inner = getattr(ops, name)

        def wrapper(*args, **kw):
            self.seen.append(note(*args, **kw))
            return inner(*args, **kw)
        monkeypatch.setattr(ops, name, wrapper)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", ["whole", "tail", "ragged", "mixed"])
@pytest.mark.parametrize("key", ["a", "b", "c", "d", "ds", "e"])
def test_replay_matches_plain(model_dirs, plain_cache, key, cut, dtype):
    raw, reqs, want = _plain(plain_cache, key, model_dirs[key])
    steps = CUTS[cut](reqs)
    runner = _runner(model_dirs[key], dtype, SETUP[key][0], steps)
    got = ru.run_trace(runner, steps)
    assert len(got) == sum(len(t) for t in reqs.values())
    ru.compare(got, want, dtype, label=f"{key}/{cut}/{dtype}")
    runner.cache.check_consistency()
    assert runner.cache.num_free_pages(0) == runner.cache.pools[0].num_pages


def _wide_requests(raw, n_live, tail, seed):
    import random
    rng = random.Random(seed)
    lens = [rng.randint(tail + 2, tail + 50) for _ in range(n_live)] + [tail + 18, tail + 27] + \
           [rng.randint(tail + 2, tail + 50) for _ in range(n_live)]
    return {f"w{i}": random_tokens(raw["vocab_size"], n, seed * 1000 + i) for i, n in enumerate(lens)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_live", [12, 33, 64])
@pytest.mark.parametrize("key", ["ds", "e"])
def test_wide_decode_batches_match_plain(model_dirs, monkeypatch, key, n_live, dtype):
    """12, 33 and 64 requests decoding together, prompt portions of others beside them in some
    steps, a second group that takes over the first group's pages: with more than eight rows every
    projection leaves the skinny kernel for the library product (or the swapped-operand kernel) with
    stand-alone norm, rotary and activation kernels, and the decode attention runs with many rows.
    Logits at every position against the plain implementation, and a check that those routes ran."""
    raw, w = load_plain(model_dirs[key])
    tail = 12
    reqs = _wide_requests(raw, n_live, tail, seed=n_live)
    steps = ru.wide(reqs, n_live, tail=tail)
    assert sum(1 for s in steps if len(s["entries"]) >= n_live and all(len(e["tokens"]) == 1 for e in s["entries"])) >= tail
    decode_rows = _Spy(monkeypatch, "attention_decode", lambda *a, **k: a[5])          # n_items
    library_rows = _Spy(monkeypatch, "linear_bf16", lambda x, *a, **k: x.shape[0])
    plain_rows = _Spy(monkeypatch, "attention_generic", lambda q, *a, **k: q.shape[0])
    runner = _runner(model_dirs[key], dtype, 16, steps, max_requests=n_live + 2)
    got = ru.run_trace(runner, steps)
    assert len(got) == sum(len(t) for t in reqs.values())
    ru.compare(got, ru.plain_logits(raw, w, reqs), dtype, label=f"wide/{key}/{n_live}/{dtype}")
    runner.cache.check_consistency()
    assert runner.cache.num_free_pages(0) == runner.cache.pools[0].num_pages
    if dtype == "bfloat16":
        assert max(decode_rows.seen) >= n_live, "the split-K decode attention never saw the whole batch"
        assert max(library_rows.seen) >= n_live, "no projection of the whole batch went to the library product"
        assert any(n >= n_live for n in runner._graphs), "steps of n_live single tokens are expected to be captured and replayed"
    else:
        assert max(plain_rows.seen) >= n_live


@pytest.mark.parametrize("key", ["ds", "e"])
def test_wide_decode_batches_with_the_balanced_attention(model_dirs, monkeypatch, key):
    """The same kind of trace with the single-token attention on the kernel that deals all tokens' keys
    evenly over a fixed grid (the default for wide heads and many tokens; switched on here for these
    small models): requests of different lengths beside one another, short portions of prompts among
    the single tokens, pages that come back, steps replayed from graphs."""
    raw, w = load_plain(model_dirs[key])
    n_live, tail = 33, 12
    reqs = _wide_requests(raw, n_live, tail, seed=77)
    steps = ru.wide(reqs, n_live, tail=tail)
    balanced_rows = _Spy(monkeypatch, "attention_decode_balanced", lambda *a, **k: a[5])
    split_rows = _Spy(monkeypatch, "attention_decode", lambda *a, **k: a[5])
    runner = _runner(model_dirs[key], "bfloat16", 16, steps, max_requests=n_live + 2)
    runner.rt.balanced_attention_pairs, runner.rt.balanced_attention_narrow_heads = 2, True
    got = ru.run_trace(runner, steps)
    assert len(got) == sum(len(t) for t in reqs.values())
    ru.compare(got, ru.plain_logits(raw, w, reqs), "bfloat16", label=f"balanced/{key}")
    runner.cache.check_consistency()
    assert max(balanced_rows.seen) >= n_live and any(n >= n_live for n in runner._graphs)
    assert all(n * raw["num_key_value_heads"] <= 2 for n in split_rows.seen)     # only the smallest steps took the split kernel


@pytest.mark.parametrize("key", ["ds", "e"])
def test_single_token_steps_hand_their_norms_from_kernel_to_kernel(model_dirs, plain_cache, monkeypatch, key):
    """In steps of up to 8 rows the product that adds into the residual stream prepares the norm that
    follows, and gate/up and the QKV projection read it prepared: only the output projection over the
    vocabulary still runs a norm inside itself.  Logits against the plain implementation, and - to
    rounding - against the same run with the hand-over switched off."""
    from nanoinfer_b200.kernels import ops
    raw, reqs, want = _plain(plain_cache, key, model_dirs[key])
    page = SETUP[key][0]
    steps = ru.tail_by_token(reqs)
    readers = _Spy(monkeypatch, "gemv_bf16", lambda x, w, out, mode, *a, **k: k.get("pre") is not None)
    qkv_readers = _Spy(monkeypatch, "gemv_qkv_rope", lambda *a, **k: k.get("pre") is not None)
    inside = _Spy(monkeypatch, "gemv_norm_bf16", lambda h, gain, eps, rows, w, *a, **k: w.shape[0])
    runner = _runner(model_dirs[key], "bfloat16", page, steps)
    got = ru.run_trace(runner, steps)
    ru.compare(got, want, "bfloat16", label=f"handoff/{key}")
    assert sum(readers.seen) > 0 and sum(qkv_readers.seen) > 0
    n_layers = raw["num_hidden_layers"]
    # per single-token step: every gate/up reads a prepared norm, and every QKV projection but the first layer's
    assert sum(readers.seen) * (n_layers - 1) == sum(qkv_readers.seen) * n_layers
    assert set(inside.seen) <= {raw["vocab_size"], 2 * raw["intermediate_size"]}      # (gate/up of the prompt's last portion may be skinny too)
    runner2 = _runner(model_dirs[key], "bfloat16", page, steps)
    runner2.rt.norm_handoff = False
    got2 = ru.run_trace(runner2, steps)
    worst = max((got[k] - got2[k]).abs().max().item() / max(got2[k].abs().max().item(), 1e-6) for k in got)
    assert worst <= 0.02, f"with and without the hand-over the logits differ by {worst:.3g} of their size"


@pytest.mark.parametrize("every_projection", [False, True])
def test_wide_outputs_take_the_swapped_operand_product(model_dirs, monkeypatch, every_projection):
    """A vocabulary wide enough that, at 9 to 128 rows, the output projection goes to the
    swapped-operand tcgen05 kernel (one thin layer, so the plain implementation stays quick).  With
    every projection routed there (an option; the library product is the default for the layers'
    own projections), each of its fused epilogues - rotation and cache write, addition into the
    residual stream, the gated activation - serves the same logits."""
    from nanoinfer_b200.engine.runtime import Runtime
    from nanoinfer_b200.kernels import ops
    raw, w = load_plain(model_dirs["f"])
    n_live, tail = 12, 6
    reqs = _wide_requests(raw, n_live, tail, seed=5)
    steps = ru.wide(reqs, n_live, tail=tail)
    swapped = _Spy(monkeypatch, "gemm_swap_tc", lambda x, w_, out, mode, *a, **k: (x.shape[0], mode))
    runner = _runner(model_dirs["f"], "bfloat16", 16, steps, max_requests=n_live + 2)
    if every_projection:
        runner.rt.mid_batch_mask = (Runtime.MID_QKV | Runtime.MID_OUT | Runtime.MID_GATE_UP | Runtime.MID_DOWN
                                    | Runtime.MID_HEAD)
    got = ru.run_trace(runner, steps)
    ru.compare(got, ru.plain_logits(raw, w, reqs), "bfloat16", label="wide/f")
    ops.check_device_errors()
    modes = {m for _, m in swapped.seen}
    assert ops.STORE_F32 in modes, "the output projection over the vocabulary did not take the swapped-operand kernel"
    layer_modes = {ops.ROPE_KV, ops.ADD_F32, ops.SWIGLU_BF16}
    assert (layer_modes <= modes) if every_projection else not (layer_modes & modes)
    assert max(r for r, _ in swapped.seen) >= n_live


def test_repeated_portion_shapes_are_replayed_from_a_graph(model_dirs, plain_cache):
    """Portions of one size, step after step (the way a scheduler cuts prompts): from the second
    appearance (as set here) the step is a replayed graph; the logits must not notice, also when the same graph
    serves another request, another position in the cache and a portion beside a decoded token."""
    key = "d"
    raw, reqs, want = _plain(plain_cache, key, model_dirs[key])
    page = SETUP[key][0]
    steps, s = [], 0
    items = list(reqs.items())
    for rid, toks in items[:3]:                       # one request at a time, portions of 24
        for at in range(0, len(toks), 24):
            n = min(24, len(toks) - at)
            steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[at:at + n], "want": list(range(n))}],
                          "end": [rid] if at + n == len(toks) else []})
            s += 1
    (ra, ta), (rb, tb) = items[3], items[4]           # a portion of one beside single tokens of another
    steps.append({"step": s, "entries": [{"id": rb, "tokens": tb[:40], "want": list(range(40))}], "end": []})
    s += 1
    at_a, at_b = 0, 40
    while at_a < len(ta):
        n = min(16, len(ta) - at_a)
        entries = [{"id": ra, "tokens": ta[at_a:at_a + n], "want": list(range(n))}]
        if at_b < len(tb):
            entries.append({"id": rb, "tokens": [tb[at_b]], "want": [0]})
            at_b += 1
        at_a += n
        steps.append({"step": s, "entries": entries, "end": [ra] if at_a == len(ta) else []})
        s += 1
    while at_b < len(tb):
        steps.append({"step": s, "entries": [{"id": rb, "tokens": [tb[at_b]], "want": [0]}], "end": []})
        at_b += 1
        s += 1
    steps[-1]["end"] = [rb]
    runner = _runner(model_dirs[key], "bfloat16", page, steps)
    runner.portion_graph_after = 2
    got = ru.run_trace(runner, steps)
    assert len(got) == sum(len(t) for t in reqs.values())
    ru.compare(got, want, "bfloat16", label="portion graphs")
    assert any(sig == ((24, 24),) for sig in runner._portion_graphs) and any(len(sig) == 2 for sig in runner._portion_graphs)
    assert runner.cache.num_free_pages(0) == runner.cache.pools[0].num_pages


def test_more_recurring_step_shapes_than_graph_places_do_not_take_turns(model_dirs, plain_cache, monkeypatch):
    """Four portion sizes come round and round while the runner keeps two captured shapes: the first
    two are captured and replayed, the others run without a graph - no capture per step.  Once a
    captured shape has stayed away long enough, a new one takes its place.  The logits do not notice."""
    from nanoinfer_b200.engine import step as step_module
    key = "d"
    raw, reqs, want = _plain(plain_cache, key, model_dirs[key])
    page = SETUP[key][0]
    rid, toks = max(reqs.items(), key=lambda kv: len(kv[1]))          # the longest request, in portions of 5, 6, 7, 8, 5, ...
    steps, at, s = [], 0, 0
    while at < len(toks):
        n = min(5 + s % 4, len(toks) - at)
        steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[at:at + n], "want": list(range(n))}],
                      "end": [rid] if at + n == len(toks) else []})
        at, s = at + n, s + 1
    assert len(steps) > 40
    captured = []
    init = step_module._PortionGraph.__init__

    def counting_init(self, runner):
        captured.append(runner._step_no)
        init(self, runner)
    monkeypatch.setattr(step_module._PortionGraph, "__init__", counting_init)
    runner = _runner(model_dirs[key], "bfloat16", page, steps)
    runner.portion_graph_after, runner.max_portion_graphs = 2, 2
    got = ru.run_trace(runner, steps)
    ru.compare(got, {rid: want[rid]}, "bfloat16", label="graph places")
    assert len(captured) == 2 and len(runner._portion_graphs) == 2, f"captures at steps {captured}"
    # a shape that has stayed away for portion_graph_idle steps gives way
    runner2 = _runner(model_dirs[key], "bfloat16", page, steps)
    runner2.portion_graph_after, runner2.max_portion_graphs, runner2.portion_graph_idle = 2, 2, 3
    captured.clear()
    got2 = ru.run_trace(runner2, steps)
    ru.compare(got2, {rid: want[rid]}, "bfloat16", label="graph places, short idle time")
    assert len(captured) > 2


@pytest.mark.parametrize("key", ["a", "b", "e"])
def test_cuts_agree_bitwise_in_float32(model_dirs, plain_cache, key):
    """The 32-bit path fixes the order of every sum, so the cut cannot change a single bit."""
    raw, reqs, _ = _plain(plain_cache, key, model_dirs[key])
    results = {}
    for cut, fn in CUTS.items():
        steps = fn(reqs)
        results[cut] = ru.run_trace(_runner(model_dirs[key], "float32", SETUP[key][0], steps), steps)
    for cut in ("tail", "ragged", "mixed"):
        for k, row in results["whole"].items():
            assert torch.equal(row, results[cut][k]), f"{key}: {cut} differs from whole at {k}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_dirs, dtype):
    """A short prompt and then hundreds of tokens one by one (captured decode steps, pages
    taken one at a time), against the plain implementation at every position."""
    raw, w = load_plain(model_dirs["d"])
    reqs = {"long": random_tokens(raw["vocab_size"], 420, 11), "other": random_tokens(raw["vocab_size"], 300, 12)}
    steps = ru.tail_by_token(reqs, tail=290)
    runner = _runner(model_dirs["d"], dtype, 16, steps)
    got = ru.run_trace(runner, steps)
    ru.compare(got, ru.plain_logits(raw, w, reqs), dtype, label=f"long/{dtype}")
    assert runner._graphs, "single-token steps are expected to run as captured graphs"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["a", "b", "d"])
def test_first_tokens_of_a_sequence(model_dirs, key, dtype):
    """Positions 0, 1, 2: one key, two keys; alone, token by token and as a batch of short requests."""
    raw, w = load_plain(model_dirs[key])
    reqs = {f"s{n}": random_tokens(raw["vocab_size"], n, 20 + n) for n in (1, 2, 3, 4)}
    want = ru.plain_logits(raw, w, reqs)
    page = SETUP[key][0]
    for steps in (ru.whole(reqs), ru.tail_by_token(reqs, tail=4),
                  [{"step": 0, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in reqs.items()],
                    "end": list(reqs)}]):
        got = ru.run_trace(_runner(model_dirs[key], dtype, page, steps), steps)
        ru.compare(got, want, dtype, label=f"first/{key}/{dtype}")


def test_trace_run_program(model_dirs, tmp_path):
    """bin/trace_run as a user runs it: JSON lines in, <step>.f32 files and 'done' lines out."""
    raw, w = load_plain(model_dirs["a"])
    reqs = _requests(raw, [33, 70, 20], seed=7)
    steps = ru.mixed(reqs, max_live=2)
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dirs["a"], "--dtype",
         "float32", "--out", str(out), "--max-tokens", str(ru.max_live_tokens(steps, 64))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    want = ru.plain_logits(raw, w, reqs)
    fed = {}
    for s in steps:
        n_want = sum(len(e["want"]) for e in s["entries"])
        path = out / f"{s['step']}.f32"
        if n_want == 0:
            assert not path.exists()
            continue
        logits = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(n_want, raw["vocab_size"]))
        r = 0
        for e in s["entries"]:
            base = fed.get(e["id"], 0)
            for wpos in e["want"]:
                torch.testing.assert_close(logits[r], want[e["id"]][base + wpos], rtol=ru.F32_RTOL, atol=ru.F32_ATOL)
                r += 1
            fed[e["id"]] = base + len(e["tokens"])


def test_replay_goes_past_the_models_position_limit_and_serving_does_not(model_dirs, tmp_path):
    """Tiny A says max_position_embeddings 128.  Replay feeds the tokens it is given all the same (positions are
    computed, no table ends at the limit) and says so once on standard error; the logits past the limit
    are the plain implementation's.  A runner built for serving refuses the step that would pass the limit."""
    from nanoinfer_b200.engine import StepEntry, StepError
    raw, w = load_plain(model_dirs["a"])
    assert raw["max_position_embeddings"] == 128
    reqs = _requests(raw, [150, 40], seed=8)
    steps = ru.ragged(reqs)
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dirs["a"], "--dtype",
         "float32", "--out", str(out), "--max-tokens", str(ru.max_live_tokens(steps, 64))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stderr.count("max_position_embeddings") == 1
    want = ru.plain_logits(raw, w, reqs)
    fed, checked_past = {}, 0
    for s in steps:
        n_want = sum(len(e["want"]) for e in s["entries"])
        if n_want == 0:
            continue
        logits = torch.from_numpy(np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(n_want, raw["vocab_size"]))
        r = 0
        for e in s["entries"]:
            base = fed.get(e["id"], 0)
            for wpos in e["want"]:
                torch.testing.assert_close(logits[r], want[e["id"]][base + wpos], rtol=ru.F32_RTOL, atol=ru.F32_ATOL)
                checked_past += base + wpos >= 128
                r += 1
            fed[e["id"]] = base + len(e["tokens"])
    assert checked_past == 150 - 128
    runner = _runner(model_dirs["a"], "float32", 16, steps)
    runner.step([StepEntry("x", reqs["r0"][:128], [127])])
    with pytest.raises(StepError, match="limit of 128"):
        runner.step([StepEntry("x", reqs["r0"][128:130], [1])])


_LAYER_SIZES = {
    # width, q heads, kv heads, head size, feed-forward, vocabulary, rope factor, tied output
    "1b": (2048, 32, 8, 64, 8192, 128256, 32.0, True),
    "3b": (3072, 24, 8, 128, 8192, 32064, 32.0, True),      # odd group of 3, a width that is no power of two
    "8b": (4096, 32, 8, 128, 14336, 32064, 8.0, False),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", sorted(_LAYER_SIZES))
def test_benchmark_layer_sizes(tmp_path_factory, dtype, shape):
    """The layer sizes of the family's models (1B: width 2048, 32/8 heads of 64, feed-forward 8192,
    vocabulary 128256, tied output; 3B and 8B: heads of 128, with a smaller vocabulary to keep the
    plain implementation quick), llama3 rope scaling, two layers: a prompt long enough for the
    tensor-core projection path, then single tokens through the captured decode step."""
    from nanoinfer_b200.weights import write_random_model
    width, hq, hkv, hd, inter, vocab, factor, tied = _LAYER_SIZES[shape]
    raw = {"architectures": ["LlamaForCausalLM"], "hidden_size": width, "intermediate_size": inter,
           "num_hidden_layers": 2, "num_attention_heads": hq, "num_key_value_heads": hkv, "head_dim": hd,
           "vocab_size": vocab, "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 8192},
           "tie_word_embeddings": tied, "hidden_act": "silu"}
    d = str(tmp_path_factory.mktemp("bench_shape") / "m")
    write_random_model(d, raw, seed=4)
    raw_read, w = load_plain(d)
    toks = random_tokens(raw["vocab_size"], 300, 5)
    want = {"p": ru.plain_logits(raw_read, w, {"p": toks})["p"]}
    steps = [{"step": 0, "entries": [{"id": "p", "tokens": toks[:290], "want": [0, 100, 289]}], "end": []}]
    steps += [{"step": 1 + i, "entries": [{"id": "p", "tokens": [toks[290 + i]], "want": [0]}],
               "end": ["p"] if i == 9 else []} for i in range(10)]
    runner = _runner(d, dtype, 16, steps)
    got = ru.run_trace(runner, steps)
    assert len(got) == 13
    ru.compare(got, want, dtype, label=f"layer-sizes-{shape}/{dtype}")
    from nanoinfer_b200.kernels import ops
    ops.check_device_errors()


@pytest.mark.parametrize("key", ["ds", "e"])
def test_a_wrong_page_breaks_the_bfloat16_bound(model_dirs, key):
    """The bfloat16 tolerances must bite: with one entry of one request's block table pointing at
    another request's page (a valid page of the pool, injected on the host), the logits of the next
    decoded token have to fall outside them.  The same steps with the true table pass.  (Models with
    peaked attention: with the near-uniform attention of N(0, 0.02) projections sixteen wrong keys
    among a hundred would move the logits by less than bfloat16 rounding does.)"""
    raw, w = load_plain(model_dirs[key])
    reqs = {"x": random_tokens(raw["vocab_size"], 100, 31), "y": random_tokens(raw["vocab_size"], 90, 32)}
    want = ru.plain_logits(raw, w, reqs)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": reqs["x"][:99], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "y", "tokens": reqs["y"], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": reqs["x"][99:], "want": [0]}], "end": ["x", "y"]}]
    for wrong in (False, True):
        runner = _runner(model_dirs[key], "bfloat16", 16, steps)
        if wrong:
            true_rows = runner.cache.table_rows

            def swapped(group, slots, width=None, true_rows=true_rows, cache=runner.cache):
                rows = true_rows(group, slots, width).copy()
                if cache.has("x") and cache.has("y") and cache.length("x") == 100:
                    for i, s in enumerate(slots):
                        if s == cache.slot("x"):
                            rows[i, 2] = true_rows(group, [cache.slot("y")], width)[0, 2]   # tokens 32..47 of the other request
                return rows
            runner.cache.table_rows = swapped
        got = ru.run_trace(runner, steps)
        assert list(got) == [("x", 99)]
        if wrong:
            with pytest.raises(AssertionError):
                ru.compare(got, want, "bfloat16", label="wrong page")
        else:
            ru.compare(got, want, "bfloat16", label="true pages")


@pytest.mark.slow
def test_full_size_model_in_float32_all_cuts(tmp_path_factory):
    """All 16 layers of the 1B configuration (the package's own config.json of that size, random
    weights) in true 32-bit: three requests through the four cuts with reused pages.  Logits at every
    position against the plain implementation, the cuts bitwise equal among themselves, and a greedy
    continuation equal to the plain one.  (About 5 GB of weights on the host and on the device; the
    plain implementation runs ~1.5 TFLOP on the CPU.)"""
    from nanoinfer_b200.config import preset
    from nanoinfer_b200.weights import write_random_model
    import plain_llama as plain
    raw = preset("llama-3.2-1b")
    assert raw["num_hidden_layers"] == 16 and raw["vocab_size"] == 128256
    d = str(tmp_path_factory.mktemp("full_size") / "m")
    s = (1.5 / raw["hidden_size"]) ** 0.5
    write_random_model(d, raw, seed=9, slot_std={"q": s, "k": s})
    raw_read, w = load_plain(d)
    reqs = {"p": random_tokens(raw["vocab_size"], 280, 1), "q": random_tokens(raw["vocab_size"], 130, 2),
            "r": random_tokens(raw["vocab_size"], 75, 3)}
    # At this size two correct 32-bit computations that add in different orders no longer agree to the
    # 1e-4 of the small models (sums of 8,192 terms, 16 layers).  The yardstick is therefore the
    # plain implementation itself: its 32-bit result against its 64-bit result is how far a 32-bit
    # computation of this model is from the exact one; the engine may be no further than a small
    # multiple of that, at any logit of any position.
    want32 = ru.plain_logits(raw_read, w, reqs)
    with plain.precision(torch.float64):
        want64 = ru.plain_logits(raw_read, w, reqs)
    plain_error = max((want32[r].double() - want64[r]).abs().max().item() for r in reqs)
    scale = max(want64[r].abs().max().item() for r in reqs)
    assert plain_error < 1e-4 * scale, "the 32-bit plain implementation itself is off"
    results = {}
    for cut, fn in CUTS.items():
        steps = fn(reqs) if cut != "mixed" else ru.mixed(reqs, max_live=2)     # two live: the third takes over freed pages
        runner = _runner(d, "float32", 16, steps)
        got = ru.run_trace(runner, steps)
        assert len(got) == sum(len(t) for t in reqs.values())
        engine_error = max((row.double() - want64[rid][pos]).abs().max().item() for (rid, pos), row in got.items())
        # (The engine adds each dot product's terms one after the other in ascending order, so that no
        # cut can change a bit; the CPU library adds 16 lanes side by side.  One chain of 8,192 terms
        # rounds about sqrt(16) = 4 times as much as 16 chains of 512: measured 4.2.  Twice that is allowed.)
        assert engine_error <= 8.0 * plain_error, \
            f"1b/{cut}: engine {engine_error:.3g} from the exact logits, the plain 32-bit computation {plain_error:.3g}"
        results[cut] = got
        runner.cache.check_consistency()
        del runner
        torch.cuda.empty_cache()
    for cut in ("tail", "ragged", "mixed"):
        for k, row in results["whole"].items():
            assert torch.equal(row, results[cut][k]), f"1b: {cut} differs from whole at {k}"
    # greedy continuation: the engine's tokens are the plain implementation's
    from nanoinfer_b200 import Engine, SamplingParams
    prompt = reqs["r"][:20]
    eng = Engine.from_model_dir(d, dtype="float32", block_size=16, num_cache_blocks=16, max_sequences=2)
    eng.stop_token_ids = ()
    assert eng.generate([prompt], max_new_tokens=5, sampling_params=SamplingParams.greedy())[0] == \
        plain.greedy_generate(raw_read, w, prompt, 5)
