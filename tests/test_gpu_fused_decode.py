"""The fused decode step (one persistent kernel for a step of up to 8 single tokens) against the
plain implementation and against the same engine with the step run part by part."""
import pytest
import torch

import replay_util as ru
from helpers import load_plain, random_tokens

pytestmark = pytest.mark.gpu


def _runner(model_dir, page, num_pages, fused):
    from nanoinfer_b200.config import load_config
    from nanoinfer_b200.engine import ModelRunner
    from nanoinfer_b200.weights import load_weights
    cfg = load_config(model_dir)
    return ModelRunner(cfg, load_weights(model_dir, cfg), dtype="bfloat16", page_size=page, num_pages=num_pages,
                       max_requests=8, fused_decode=fused)


def _decode_trace(reqs, tail):
    """Every request's prompt whole, one per step; then all requests one token per step, together."""
    steps = []
    for rid, toks in reqs.items():
        head = len(toks) - tail
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head], "want": [head - 1]}], "end": []})
    for j in range(tail):
        entries = [{"id": rid, "tokens": [toks[len(toks) - tail + j]], "want": [0]} for rid, toks in reqs.items()]
        steps.append({"step": len(steps), "entries": entries, "end": list(reqs) if j == tail - 1 else []})
    return steps


@pytest.mark.parametrize("lens", [[70], [33, 5, 130], [64, 65, 17, 200, 3, 129, 90, 48]])
@pytest.mark.parametrize("key,page", [("ds", 16), ("e", 16), ("e", 8), ("bs", 8)])
def test_fused_decode_step_matches_plain_and_the_parts(model_dirs, monkeypatch, key, page, lens):
    """1, 3 and 8 requests decoding together after prompts of different lengths (contexts that end
    inside a page, at a page's edge, in the first page).  "ds": heads of 64, inner sizes that are
    8 mod 16; "e": heads of 128 in groups of three; "bs" has heads of 32, which the kernel does
    not take: it must be left to the parts, silently."""
    from nanoinfer_b200.kernels import ops
    raw, w = load_plain(model_dirs[key])
    tail = 7
    reqs = {f"r{i}": random_tokens(raw["vocab_size"], n + tail, 700 + i) for i, n in enumerate(lens)}
    steps = _decode_trace(reqs, tail)
    want = ru.plain_logits(raw, w, reqs)
    calls = []
    inner = ops.decode_fused
    monkeypatch.setattr(ops, "decode_fused", lambda p: (calls.append((p.M, p.R)), inner(p))[1])
    pages = ru.max_live_tokens(steps, 64) // page
    got = ru.run_trace(_runner(model_dirs[key], page, pages, True), steps)
    ops.check_device_errors()
    ru.compare(got, want, "bfloat16", label=f"fused/{key}")
    if raw["head_dim"] in (64, 128):
        assert calls and all(c == (len(lens), len(lens)) for c in calls), "single-token steps were expected to run fused"
    else:
        assert not calls
    n_fused = len(calls)
    parts = ru.run_trace(_runner(model_dirs[key], page, pages, False), steps)
    assert len(calls) == n_fused, "with the fused step switched off the parts must run"
    # the two routes round differently here and there (bfloat16 activations between the parts'
    # kernels, the same inside the fused one): they must agree far better than either must with FP32
    for k, row in got.items():
        ref = parts[k]
        assert (row - ref).abs().max().item() <= 0.02 * ref.abs().max().item(), f"fused vs parts at {k}"


def test_fused_decode_at_the_model_sizes(tmp_path):
    """Two layers of the 1B sizes (width 2048, 32/8 heads of 64, feed-forward 8192, vocabulary
    128256, tied, llama3 rope scaling): 8 requests at contexts around 300, fused step against plain."""
    from nanoinfer_b200.weights import write_random_model
    raw = {"architectures": ["LlamaForCausalLM"], "hidden_size": 2048, "intermediate_size": 8192,
           "num_hidden_layers": 2, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
           "vocab_size": 128256, "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 8192},
           "tie_word_embeddings": True, "hidden_act": "silu"}
    d = str(tmp_path / "m")
    write_random_model(d, raw, seed=8, slot_std={"q": 0.027, "k": 0.027})
    raw_read, w = load_plain(d)
    tail = 4
    reqs = {f"r{i}": random_tokens(raw["vocab_size"], n + tail, 900 + i) for i, n in enumerate([300, 17, 129, 256, 64, 511, 1, 90])}
    steps = _decode_trace(reqs, tail)
    runner = _runner(d, 16, ru.max_live_tokens(steps, 64) // 16, True)
    got = ru.run_trace(runner, steps)
    from nanoinfer_b200.kernels import ops
    ops.check_device_errors()
    assert runner.model._fused is not None
    ru.compare(got, ru.plain_logits(raw_read, w, reqs), "bfloat16", label="fused/1b-sizes")


def test_a_grid_barrier_that_is_never_complete_is_given_up(model_dirs):
    """Block 0 leaves out one arrival (a switch of the kernel for this test), so one grid barrier
    can never be passed: every block's wait runs out after about a millisecond, the kernel records
    it and returns, the error reaches the host, and the next step is an ordinary one."""
    from nanoinfer_b200.engine import StepEntry
    from nanoinfer_b200.kernels import ops
    raw, w = load_plain(model_dirs["ds"])
    runner = _runner(model_dirs["ds"], 16, 32, True)
    runner.use_graphs = False
    toks = random_tokens(raw["vocab_size"], 40, 5)
    want = ru.plain_logits(raw, w, {"r": toks})["r"]
    runner.step([StepEntry("r", toks[:30], [])])
    logits = runner.step([StepEntry("r", toks[30:31], [0])]).cpu()
    ru.compare({("r", 30): logits[0]}, {"r": want}, "bfloat16")
    fused = runner.model._fused
    fused.params.wait_limit, fused.params.skip_arrive_at = 2_000_000, 4
    runner.step([StepEntry("r", toks[31:32], [0])])
    torch.cuda.synchronize()                       # returns: nothing spins without a bound
    with pytest.raises(ops.KernelError, match="code 31"):
        ops.check_device_errors()
    fused.params.wait_limit, fused.params.skip_arrive_at = 0, -1
    runner.end("r")                                # what that step wrote is not to be trusted: start over
    runner.step([StepEntry("r", toks[:32], [])])
    logits = runner.step([StepEntry("r", toks[32:33], [0])]).cpu()
    ops.check_device_errors()
    ru.compare({("r", 32): logits[0]}, {"r": want}, "bfloat16")
