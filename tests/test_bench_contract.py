"""What of bench.py's contract can be checked without a GPU: the reference arm's line, the refusal of
more than one GPU, the byte and FLOP counts that the roofline fractions are made from, and the clock
sampler's summary."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _run(*args, env=None):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=300, env=dict(os.environ, **(env or {})))


def test_reference_arm_prints_one_json_line_and_exits_0():
    p = _run("--impl", "reference", "--gpus", "1", "--steps", "5", "--warmup", "3")
    assert p.returncode == 0
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and isinstance(rec["unavailable"], str) and "\n" not in rec["unavailable"]


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_2():
    p = _run("--gpus", "2", "--steps", "5", "--warmup", "3")
    assert p.returncode == 2 and len(p.stdout.strip().splitlines()) == 1
    p = _run("--steps", "5", env={"WORLD_SIZE": "4"})          # launched as one of several ranks
    assert p.returncode == 2


def test_byte_and_flop_counts_of_the_1b_shape():
    """2.47 GB of bfloat16 weights per decode step, 32 KiB of keys and values per token, 4.26 TFLOP for a
    prompt of 2,048 tokens: the figures the roofline fractions divide by, recomputed from the config alone."""
    b = _bench()
    raw = b.shape_config("llama-3.2-1b")
    nums = b.model_numbers(raw, raw["num_hidden_layers"])
    d, ff, hq, hkv, hd, v, n = (raw["hidden_size"], raw["intermediate_size"], raw["num_attention_heads"],
                                raw["num_key_value_heads"], raw["head_dim"], raw["vocab_size"], raw["num_hidden_layers"])
    per_layer = d * (hq + 2 * hkv) * hd + hq * hd * d + 3 * d * ff
    assert nums["linear_params"] == n * per_layer
    assert nums["lm_head_params"] == v * d
    assert nums["kv_bytes_per_token"] == n * 2 * hkv * hd * 2 == 32768
    weight_bytes = 2.0 * (nums["linear_params"] + nums["lm_head_params"]) + 4.0 * nums["norm_params"]
    assert abs(weight_bytes / 1e9 - 2.4715) < 2e-3
    t = 2048
    flops = 2.0 * t * nums["linear_params"] + nums["attn_flops_per_key_query"] * t * (t + 1) / 2 + 2.0 * nums["lm_head_params"]
    assert abs(flops / 1e12 - 4.26) < 0.03


def test_peaks_come_from_the_measured_file_when_it_is_there():
    b = _bench()
    pk = b.peaks()
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            m = json.load(f)
        assert pk["source"] == "measured" and pk["hbm_gbs"] == m["hbm_gbs"] and pk["bf16_tflops"] == m["bf16_tflops"]
    else:
        assert pk["source"] == "fallback" and pk["hbm_gbs"] == 6650.0 and pk["bf16_tflops"] == 1590.0
