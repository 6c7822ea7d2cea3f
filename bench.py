#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the Llama 3.2 1B shape with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers 16] [--impl ours|reference]

A "step" is one decode step of the whole batch.  Every request starts at a context of 2,048
tokens and decodes W + K tokens (by default to 4,096).  Prints ONE JSON line:
  value      decoded tokens per second, timed on the device with CUDA events over exactly K
             replays of the captured decode step (forward pass, arg-max and token feedback all
             on the device);
  e2e        the same through the public API (Engine.step): host token ids in, host token ids
             out, every step with its pinned host-to-device metadata copy and its
             device-to-host read of the sampled ids;
  prefill    one prompt of 2,048 tokens in one step (tokens/s, share of the bf16 peak);
  roofline   bytes the decode step must read (every weight once + the live requests' cache)
             over its time, against the measured HBM bandwidth;
  points     decode tokens per second at batch 1 and 64.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The layer sizes come from the package's config.json files of the family's published sizes; the
# default run and the published line are the 1B shape, --shape names the others.
SHAPE_NAMES = ["llama-3.1-8b", "llama-3.2-1b", "llama-3.2-3b"]


def shape_config(name):
    from nanoinfer_b200.config import preset
    return preset(name)


START_CONTEXT = 2048          # tokens each request holds when decoding starts (--context overrides)
PREFILL_TOKENS = 2048
BATCHED_TOKENS = 4 * PREFILL_TOKENS     # token budget of one step of the end-to-end run
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks, load and throttle reasons with nvidia-smi from before the warm-up until
    the last timed region has ended (every 20 ms, so that even a run of a few steps is covered);
    the clock reported is the median over the samples taken under load."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,utilization.gpu")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.lines, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, loaded, mx, reasons = [], [], 0, set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                clock = int(f[0])
                mx = max(mx, int(f[1]))
            except ValueError:
                continue
            sm.append(clock)
            try:
                busy = int(f[6]) >= 50
            except ValueError:
                busy = False
            if busy:
                loaded.append(clock)
                for name, v in zip(self.NAMES, f[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        use = sorted(loaded or sm)
        return {"sm_mhz": use[len(use) // 2] if use else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm), "samples_under_load": len(loaded)}


def device_weights(config, seed, device):
    """Random weights of the configuration straight on the device: N(0, 0.02) matrices in
    bfloat16, norm gains 1.0 (the random-weights mode's rule, without the trip through a file)."""
    import torch
    from nanoinfer_b200.weights import tensor_plan
    g = torch.Generator(device=device).manual_seed(seed)
    out = {}
    for p in tensor_plan(config):
        if p.init == "ones":
            out[p.name] = torch.ones(p.shape, dtype=torch.bfloat16, device=device)
        else:
            out[p.name] = (torch.randn(p.shape, generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    return out


def model_numbers(raw, n_layers):
    d, inter, v = raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"]
    hq, hkv, hd = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"]
    linear_per_layer = d * (hq + 2 * hkv) * hd + hq * hd * d + 3 * d * inter
    return {"linear_params": n_layers * linear_per_layer, "lm_head_params": v * d,
            "norm_params": (2 * n_layers + 1) * d, "kv_bytes_per_token": n_layers * 2 * hkv * hd * 2,
            "attn_flops_per_key_query": n_layers * 4 * hq * hd}


def run_ours(args):
    import torch
    from nanoinfer_b200 import Engine, EngineConfig, SamplingParams
    from nanoinfer_b200.config import config_from_dict
    from nanoinfer_b200.engine import StepEntry
    from nanoinfer_b200.kernels import ops

    device = "cuda:0"
    torch.cuda.set_device(0)
    full = shape_config(args.shape)
    full_layers = full["num_hidden_layers"]
    if args.layers is None:
        args.layers = full_layers
    raw = dict(full, num_hidden_layers=args.layers)
    config = config_from_dict(raw)
    nums = model_numbers(raw, args.layers)
    pk = peaks()
    vocab = raw["vocab_size"]
    K, W = args.steps, args.warmup
    START_CONTEXT = args.context
    PREFILL = args.prefill_tokens
    BATCHED = max(BATCHED_TOKENS, PREFILL)
    # spare tokens: in the end-to-end run the first requests start decoding while the last
    # prompts are still being prefilled (one prefill step takes BATCHED_TOKENS of prompt)
    spare = max(16, -(-args.batch * START_CONTEXT // BATCHED) + 8)
    end_context = max(START_CONTEXT + W + K + spare, PREFILL)
    max_batch = max(args.batch, 64 if args.points else args.batch)
    page = 16
    pages_per_request = -(-end_context // page)
    ecfg = EngineConfig(max_batch_size=max_batch, max_sequences=max_batch, prefill_chunk_size=PREFILL,
                        block_size=page, num_cache_blocks=max_batch * pages_per_request + 8,
                        max_num_batched_tokens=BATCHED, max_model_len=pages_per_request * page,
                        dtype="bfloat16", device=device)
    engine = Engine.from_weights(config, device_weights(config, 0, device), ecfg)
    runner = engine.runner
    gen = torch.Generator().manual_seed(0)

    def prompt(n):
        return torch.randint(0, vocab, (n,), generator=gen).tolist()

    def timed(fn):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    clocks = ClockSampler()
    clocks.start()              # from before the first warm-up to after the last timed region

    # ---- prefill: one prompt (2,048 tokens unless asked otherwise) in one step, logits of the last place ----
    prefill_ms = []
    for i in range(5 + 3):                     # a step shape that keeps coming back is replayed from a graph
        p = prompt(PREFILL)
        ms = timed(lambda: runner.step([StepEntry(("prefill", i), p, [PREFILL - 1])]))
        runner.end(("prefill", i))
        if i >= 5:
            prefill_ms.append(ms)
    prefill_ms = sorted(prefill_ms)[len(prefill_ms) // 2]
    ops.check_device_errors(device)
    T = PREFILL
    prefill_flops = 2.0 * T * nums["linear_params"] + nums["attn_flops_per_key_query"] * T * (T + 1) / 2 \
        + 2.0 * nums["lm_head_params"]
    prefill = {"value": round(T / (prefill_ms / 1e3), 1), "tokens": T, "ms": round(prefill_ms, 3),
               "frac": round(prefill_flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}

    # ---- decode on the device: K replays of the captured step ----
    def decode_device(batch, tag):
        reqs = [(tag, i) for i in range(batch)]
        last = []
        for r in reqs:
            logits = runner.step([StepEntry(r, prompt(START_CONTEXT), [START_CONTEXT - 1])])
            last.append(int(torch.argmax(logits[0])))
        toks = runner.greedy_decode_on_device(reqs, last, W)          # warm-up (captures the graph)
        per_step = runner._decode_graph(batch).greedy_launches        # this package's kernels per replay
        last = toks[-1].tolist()
        ms = timed(lambda: runner.greedy_decode_on_device(reqs, last, K))
        ops.check_device_errors(device)      # a kernel that gave up a wait would make the time meaningless
        for r in reqs:
            runner.end(r)
        return ms, per_step

    ms_total, launches_per_step = decode_device(args.batch, "main")
    ms_per_step = ms_total / K
    value = args.batch * K / (ms_total / 1e3)
    mean_ctx = START_CONTEXT + W + (K + 1) / 2.0
    weight_bytes = 2.0 * (nums["linear_params"] + nums["lm_head_params"]) + 4.0 * nums["norm_params"]
    step_bytes = weight_bytes + args.batch * mean_ctx * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk["source"],
                "bytes_per_step": int(step_bytes)}

    points = {}
    if args.points:
        for b in (1, 64):
            ms_b, _ = decode_device(b, f"b{b}")
            points[f"decode_b{b}"] = round(b * K / (ms_b / 1e3), 1)

    # ---- end to end through Engine.step: host ids in, host ids out ----
    prompts = [prompt(START_CONTEXT) for _ in range(args.batch)]
    ids = [engine.add_request(p, W + K + spare, SamplingParams.greedy()) for p in prompts]
    engine.stop_token_ids = ()
    for rid in ids:
        engine.get_request(rid).stop_token_ids = frozenset()
    while any(engine.get_request(r).is_prefill() for r in ids):
        engine.step()
    for _ in range(W):
        engine.step()
    runner.h2d_bytes = 0
    engine.sampler.h2d_bytes = 0
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    produced = 0
    for _ in range(K):
        produced += len(engine.step())
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    clk = clocks.stop()
    ops.check_device_errors(device)
    assert produced == args.batch * K, f"end-to-end run produced {produced} tokens, expected {args.batch * K}"
    e2e = {"value": round(produced / e2e_s, 1), "unit": "tok/s", "ms_per_step": round(e2e_s / K * 1e3, 4),
           "h2d_bytes_per_step": int((runner.h2d_bytes + getattr(engine.sampler, "h2d_bytes", 0)) / K),
           "d2h_bytes_per_step": 4 * args.batch + 4}          # the sampled ids and the device's error word

    out = {
        "metric": "decode_tokens_per_second", "value": round(value, 1), "unit": "tok/s", "n_gpus": 1,
        "steps": K, "warmup": W, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": args.shape + "-shape", "global_batch": args.batch, "seq_len": end_context,
                   "parallelism": "single-gpu", "layers": args.layers, "layers_full_model": full_layers,
                   "hidden_size": raw["hidden_size"], "intermediate_size": raw["intermediate_size"],
                   "q_heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
                   "head_dim": raw["head_dim"], "vocab_size": vocab, "start_context": START_CONTEXT,
                   "kv_page_size": page, "weights": "random N(0,0.02) bf16" + (", tied" if raw["tie_word_embeddings"] else ""),
                   "l2_policy": "inputs larger than L2 (weights %.1f GB per step)" % (weight_bytes / 1e9),
                   "decode_loop": "cuda graph replay, device-side argmax and feedback"},
        "clocks": clk, "e2e": e2e, "gpu_launches": launches_per_step * K, "prefill": prefill,
        "roofline": roofline, "points": points,
    }
    print(json.dumps(out))
    return 0


# Serving workloads through the public entry point: every request is queued at time zero and the
# scheduler takes it from there (admission, prompts in portions under the token budget, decoding).
WORKLOADS = {
    # continuous batching: prompts of mixed length, sampled tokens
    "continuous": {"shape": "llama-3.2-3b", "requests": 32, "prompt": (128, 2048), "new_tokens": 256,
                   "temperature": 0.8, "chunk": 512, "budget": 2048},
    # long prompts and long greedy decoding at a large batch
    "long": {"shape": "llama-3.1-8b", "requests": 64, "prompt": (6144, 6144), "new_tokens": 2048,
             "temperature": 0.0, "chunk": 2048, "budget": 8192},
    # a small batch of the 1B shape that samples with temperature, top-k and top-p: what the sampler costs
    "sampled": {"shape": "llama-3.2-1b", "requests": 8, "prompt": (1024, 2048), "new_tokens": 512,
                "temperature": 0.8, "top_k": 50, "top_p": 0.9, "chunk": 2048, "budget": 2048},
}


def run_serving(args):
    import random
    import torch
    from nanoinfer_b200 import Engine, EngineConfig, SamplingParams
    from nanoinfer_b200.config import config_from_dict

    w = WORKLOADS[args.workload]
    shape = args.shape or w["shape"]
    full = shape_config(shape)
    full_layers = full["num_hidden_layers"]
    layers = args.layers or full_layers
    raw = dict(full, num_hidden_layers=layers)
    config = config_from_dict(raw)
    device = "cuda:0"
    torch.cuda.set_device(0)
    n_req = args.batch or w["requests"]
    rng = random.Random(0)
    lengths = [rng.randint(*w["prompt"]) for _ in range(n_req)]
    gen = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, raw["vocab_size"], (n,), generator=gen).tolist() for n in lengths]
    page = 16
    pages = sum(-(-(n + w["new_tokens"] + 1) // page) for n in lengths) + 64
    ecfg = EngineConfig(max_batch_size=n_req, max_sequences=n_req, prefill_chunk_size=w["chunk"], block_size=page,
                        num_cache_blocks=pages, max_num_batched_tokens=w["budget"],
                        max_model_len=max(lengths) + w["new_tokens"] + page, dtype="bfloat16", device=device)
    engine = Engine.from_weights(config, device_weights(config, 0, device), ecfg)
    engine.stop_token_ids = ()

    def one_pass(new_tokens):
        sp = (SamplingParams(temperature=w["temperature"], top_k=w.get("top_k", -1), top_p=w.get("top_p", 1.0), seed=1)
              if w["temperature"] > 0 else SamplingParams.greedy())
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        ids = [engine.add_request(p, new_tokens, sp) for p in prompts]
        for rid in ids:
            engine.get_request(rid).stop_token_ids = frozenset()
        first, produced, steps = {}, 0, 0
        while engine.has_work():
            outs = engine.step()
            steps += 1
            now = time.perf_counter()
            for o in outs:
                produced += 1
                first.setdefault(o.request_id, now - t0)
        torch.cuda.synchronize()
        return time.perf_counter() - t0, produced, steps, first

    one_pass(4)                                   # warm-up: libraries, graphs of the common step shapes
    clocks = ClockSampler()
    clocks.start()
    wall, produced, steps, first = one_pass(w["new_tokens"])
    clk = clocks.stop()
    assert produced == n_req * w["new_tokens"], f"{produced} tokens produced, expected {n_req * w['new_tokens']}"
    ttft = sorted(first.values())
    stats = engine.get_scheduler_stats()
    out = {
        "metric": "serving_generated_tokens_per_second", "value": round(produced / wall, 1), "unit": "tok/s",
        "n_gpus": 1, "steps": steps, "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "wall_s": round(wall, 3), "total_tokens_per_second": round((produced + sum(lengths)) / wall, 1),
        "ttft_ms": {"mean": round(1e3 * sum(ttft) / len(ttft), 1), "median": round(1e3 * ttft[len(ttft) // 2], 1),
                    "max": round(1e3 * ttft[-1], 1)},
        "preemptions": stats.num_preemptions,
        "config": {"workload": args.workload, "model": shape + "-shape", "requests": n_req, "layers": layers,
                   "layers_full_model": full_layers, "prompt_tokens_min": min(lengths),
                   "prompt_tokens_max": max(lengths), "prompt_tokens_total": sum(lengths),
                   "new_tokens": w["new_tokens"], "temperature": w["temperature"], "top_k": w.get("top_k", -1),
                   "top_p": w.get("top_p", 1.0), "prefill_chunk": w["chunk"],
                   "token_budget": w["budget"], "kv_page_size": page, "kv_pages": pages},
        "clocks": clk,
    }
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2024)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=None, help="requests (default 8; a serving workload's own count)")
    ap.add_argument("--context", type=int, default=START_CONTEXT, help="tokens per request when decoding starts")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="length of the timed prompt")
    ap.add_argument("--shape", default=None, choices=SHAPE_NAMES, help="layer sizes of the model (default: the 1B shape)")
    ap.add_argument("--workload", default="decode", choices=["decode"] + sorted(WORKLOADS),
                    help="decode: the timed decode step (the published line); the others serve a set of requests")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (both are reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", dest="points", action="store_false", help="skip the batch 1 and 64 points")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a CMake C++/CUDA project without setup.py or pyproject.toml (pip: 'not "
                          "installable'); its engine (include/nanoinfer/model/model.h, op/encode.h) needs sentencepiece, "
                          "abseil, re2, glog and armadillo, which its build downloads and this machine does not have, and "
                          "Engine::add_request takes text that it tokenises with a tokenizer file no offline source provides"}))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.workload != "decode":
        return run_serving(args)
    args.shape = args.shape or "llama-3.2-1b"
    args.batch = args.batch or 8
    if args.warmup < 3:
        args.warmup = 3
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
