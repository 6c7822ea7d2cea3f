"""Timing of single kernels at given sizes, for tuning and for profiler captures.

    python -m nanoinfer_b200.kernels.microbench gemv --m 8 --n 16384 --k 2048 --mode swiglu --norm
    python -m nanoinfer_b200.kernels.microbench gemm_swap --m 64 --n 16384 --k 2048 --mode swiglu
    python -m nanoinfer_b200.kernels.microbench attention_decode --batch 8 --context 3072
    python -m nanoinfer_b200.kernels.microbench attention_prefill --tokens 2048 --kernel tc
    python -m nanoinfer_b200.kernels.microbench gemm_swap --m 64 --n 2048 --k 2048 --mode add --milestones
    python -m nanoinfer_b200.kernels.microbench decode_fused --batch 8 --context 2048

Each case runs its kernel over several distinct copies of its inputs in turn (together
larger than the L2 cache, so every run reads from HBM), times it with CUDA events after
warm-up and prints microseconds per launch and the achieved GB/s or TFLOP/s.
"""
from __future__ import annotations

import argparse
import math

import torch

from . import ops

DEV = "cuda:0"
L2_BYTES = 126 << 20


def _time(fns, iters: int) -> float:
    """Microseconds per call, cycling through ``fns`` (one per input copy).  The launches are
    captured into one CUDA graph, so that the host's launch rate does not limit short kernels."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(iters):
            fns[i % len(fns)]()
    graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    graph.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / iters


def gemv(args) -> None:
    m, n, k = args.m, args.n, args.k
    w_bytes = n * k * 2
    copies = max(2, min(64, -(-2 * L2_BYTES // w_bytes)))
    g = torch.Generator(device=DEV).manual_seed(0)
    ws = [(torch.randn(n, k, device=DEV, generator=g) * 0.02).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(m, k, device=DEV, generator=g).to(torch.bfloat16)
    h = torch.randn(m, k, device=DEV, generator=g)
    gain = torch.ones(k, device=DEV)
    mode = {"bf16": ops.STORE_BF16, "f32": ops.STORE_F32, "add": ops.ADD_F32, "swiglu": ops.SWIGLU_BF16}[args.mode]
    if mode == ops.SWIGLU_BF16:
        out = torch.empty(m, n // 2, dtype=torch.bfloat16, device=DEV)
    else:
        out = torch.zeros(m, n, dtype=torch.bfloat16 if mode == ops.STORE_BF16 else torch.float32, device=DEV)
    if args.norm:
        fns = [lambda w=w: ops.gemv_norm_bf16(h, gain, 1e-5, None, w, out, mode) for w in ws]
    elif args.prepared:
        # the reader of a handed-over norm: bfloat16 input, 1/rms from partial sums (here: of a stand-in producer)
        class _Norm:
            fused_kind = "rmsnorm"
        hand = ops.NormHandoff(_Norm(), gain, 1e-5, m, k, args.parts, DEV)
        hand.x.copy_(x)
        hand.ssq.fill_(float(k) / hand.parts)
        fns = [lambda w=w: ops.gemv_bf16(hand.x, w, out, mode, pre=hand) for w in ws]
    elif args.ksplit:
        fns = [lambda w=w: ops.gemv_ksplit(x, w, out, mode) for w in ws]
    else:
        fns = [lambda w=w: ops.gemv_bf16(x, w, out, mode) for w in ws]
    us = _time(fns, args.iters)
    print(f"gemv{' (K split over a cluster)' if args.ksplit else ''}{' (norm prepared by the kernel before)' if args.prepared else ''} m={m} n={n} k={k} mode={args.mode} norm={args.norm}: {us:.2f} us, "
          f"{w_bytes / us / 1e3:.0f} GB/s of weights ({copies} weight copies in turn)")


def add_rmsnorm(args) -> None:
    """Residual add + RMSNorm over [rows, width]: the same buffers again and again (as between two
    products of a prompt portion, where they lie in L2) or ``--copies`` sets in turn."""
    t, d = args.rows, args.width
    g = torch.Generator(device=DEV).manual_seed(0)
    sets = [(torch.randn(t, d, device=DEV, generator=g), torch.randn(t, d, device=DEV, generator=g).to(torch.bfloat16),
             torch.empty(t, d, dtype=torch.bfloat16, device=DEV)) for _ in range(args.copies)]
    gain = torch.ones(d, device=DEV)
    fns = [lambda h=h, dl=dl, o=o: ops.add_rmsnorm(h, dl, gain, 1e-5, o) for h, dl, o in sets]
    us = _time(fns, args.iters)
    nbytes = t * d * (4 + 2 + 4 + 2)
    print(f"add_rmsnorm rows={t} width={d} copies={args.copies}: {us:.2f} us, {nbytes / us / 1e3:.0f} GB/s "
          f"(h read and written, delta read, activations written)")


def sample(args) -> None:
    """One token per row from FP32 logits by temperature, top-k, top-p: the cluster-per-row kernel, or
    with --one-block the kernel that gives a row one block."""
    n, v = args.rows, args.vocab
    g = torch.Generator(device=DEV).manual_seed(0)
    sets = [torch.randn(n, v, device=DEV, generator=g) * 3.0 for _ in range(max(2, min(8, (2 * L2_BYTES) // (n * v * 4) + 1)))]
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    temps = torch.full((n,), args.temperature, device=DEV)
    ks = torch.full((n,), args.top_k, dtype=torch.int32, device=DEV)
    ps = torch.full((n,), args.top_p, device=DEV)
    seeds = torch.arange(n, dtype=torch.int64, device=DEV)
    counters = torch.zeros(n, dtype=torch.int64, device=DEV)
    ops.sample_by_cluster(not args.one_block)
    us = _time([lambda l=l: ops.sample(l, out, temps, ks, ps, seeds, counters) for l in sets], args.iters)
    ops.sample_by_cluster(True)
    print(f"sample{' (one block per row)' if args.one_block else ' (a cluster per row)'} rows={n} vocab={v} temperature={args.temperature} "
          f"top_k={args.top_k} top_p={args.top_p}: {us:.1f} us")


def gemm(args) -> None:
    """The tcgen05 product against the library product on the same operands."""
    m, n, k = args.m, args.n, args.k
    g = torch.Generator(device=DEV).manual_seed(0)
    a = torch.randn(m, k, device=DEV, generator=g).to(torch.bfloat16)
    b = (torch.randn(n, k, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    mode = {"bf16": ops.STORE_BF16, "f32": ops.STORE_F32, "add": ops.ADD_F32, "swiglu": ops.SWIGLU_BF16}[args.mode]
    if mode == ops.SWIGLU_BF16:
        out = torch.empty(m, n // 2, dtype=torch.bfloat16, device=DEV)
    else:
        out = torch.zeros(m, n, dtype=torch.bfloat16 if mode == ops.STORE_BF16 else torch.float32, device=DEV)
    us = _time([lambda: ops.gemm_tc(a, b, out, mode, kernel=args.kernel, accumulators=args.accumulators, tile_n=args.tile_n)], args.iters)
    ops.check_device_errors()
    ref = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    us_lib = _time([lambda: torch.matmul(a, b.t(), out=ref)], args.iters)
    flops = 2.0 * m * n * k
    print(f"gemm m={m} n={n} k={k} mode={args.mode} kernel={args.kernel or 'default'}: {us:.1f} us, {flops / us / 1e6:.0f} TFLOP/s "
          f"(library product, plain store: {us_lib:.1f} us, {flops / us_lib / 1e6:.0f} TFLOP/s)")


def gemm_swap(args) -> None:
    """The swapped-operand tensor-core product (9..128 rows) against the library product; weights
    cycle through copies larger than L2."""
    m, n, k = args.m, args.n, args.k
    w_bytes = n * k * 2
    copies = max(2, min(64, -(-2 * L2_BYTES // w_bytes)))
    g = torch.Generator(device=DEV).manual_seed(0)
    ws = [(torch.randn(n, k, device=DEV, generator=g) * 0.02).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(m, k, device=DEV, generator=g).to(torch.bfloat16)
    mode = {"bf16": ops.STORE_BF16, "f32": ops.STORE_F32, "add": ops.ADD_F32, "swiglu": ops.SWIGLU_BF16}[args.mode]
    if mode == ops.SWIGLU_BF16:
        out = torch.empty(m, n // 2, dtype=torch.bfloat16, device=DEV)
    else:
        out = torch.zeros(m, n, dtype=torch.bfloat16 if mode == ops.STORE_BF16 else torch.float32, device=DEV)
    need = ops.gemm_swap_scratch(m, n, k)
    scratch = torch.empty(max(need, 1), dtype=torch.float32, device=DEV)
    tickets = torch.zeros(-(-n // 128), dtype=torch.int32, device=DEV)
    us = _time([lambda w=w: ops.gemm_swap_tc(x, w, out, mode, scratch, tickets) for w in ws], args.iters)
    ops.check_device_errors()
    ref = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    us_lib = _time([lambda w=w: torch.matmul(x, w.t(), out=ref) for w in ws], args.iters)
    if args.milestones:
        import ctypes
        lib = ops.load("gemm_swap_tc")
        lib.ni_gemm_swap_tc_set_trace.argtypes = [ctypes.c_void_p]
        lib.ni_gemm_swap_tc_set_trace.restype = None
        stamps = torch.zeros(16, dtype=torch.int64, device=DEV)
        lib.ni_gemm_swap_tc_set_trace(stamps.data_ptr())
        ops.gemm_swap_tc(x, ws[-1], out, mode, scratch, tickets)
        torch.cuda.synchronize()
        lib.ni_gemm_swap_tc_set_trace(None)
        t = stamps.cpu().tolist()
        names = ["set-up done", "epilogue waits", "accumulator complete", "accumulator read (sums sent)", "sums arrived", "end"]
        print("  one launch, block 0, microseconds after its start: " +
              "; ".join(f"{nm} {(t[i + 1] - t[0]) / 1e3:.2f}" for i, nm in enumerate(names) if t[i + 1] > 0))
    print(f"gemm_swap m={m} n={n} k={k} mode={args.mode}: {us:.2f} us, {w_bytes / us / 1e3:.0f} GB/s of weights "
          f"(library product, plain store: {us_lib:.2f} us, {w_bytes / us_lib / 1e3:.0f} GB/s; {copies} weight copies in turn)")


def attention_decode(args) -> None:
    b, ctx, hq, hkv, hd, page = args.batch, args.context, args.q_heads, args.kv_heads, args.head_dim, args.page
    pages_per_seq = -(-ctx // page)
    kv_bytes = 2 * b * ctx * hkv * hd * 2
    copies = args.copies or max(2, min(16, -(-2 * L2_BYTES // kv_bytes)))
    g = torch.Generator(device=DEV).manual_seed(0)
    n_pages = b * pages_per_seq
    caches = [(torch.randn(n_pages, hkv, page, hd, device=DEV, generator=g).to(torch.bfloat16),
               torch.randn(n_pages, hkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)) for _ in range(copies)]
    table = torch.randperm(n_pages, device=DEV, generator=g).int().view(b, pages_per_seq)
    q = torch.randn(b, hq * hd, device=DEV, generator=g).to(torch.bfloat16)
    out = torch.empty_like(q)
    positions = torch.full((b,), ctx - 1, dtype=torch.int32, device=DEV)
    seq_of = torch.arange(b, dtype=torch.int32, device=DEV)
    splits = args.splits or ops.decode_splits(b, hkv, hd, ctx)
    ops.attention_decode_cluster_merge(not args.scratch_merge)
    scratch = torch.empty(b * hq * splits * (hd + 2), dtype=torch.float32, device=DEV)
    tickets = torch.zeros(b * hkv, dtype=torch.int32, device=DEV)
    if args.ragged:      # contexts from a quarter of --context to all of it (the cache's bytes are counted as they are read)
        positions = (torch.linspace(ctx // 4, ctx, b, device=DEV).int() - 1).contiguous()
        kv_bytes = int(2 * (positions.long() + 1).sum().item() * hkv * hd * 2)
        splits = args.splits or ops.decode_splits(b, hkv, hd, ctx)
    if args.balanced:
        scratch = torch.empty(ops.attention_decode_balanced_scratch(hq, hkv, hd), dtype=torch.float32, device=DEV)
        fns = [lambda kc=kc, vc=vc: ops.attention_decode_balanced(q, kc, vc, out, None, b, positions, seq_of, table, hq, hkv,
                                                                  hd, page, None, 1.0 / math.sqrt(hd), scratch, tickets)
               for kc, vc in caches]
    else:
        scratch = torch.empty(b * hq * splits * (hd + 2), dtype=torch.float32, device=DEV)
        fns = [lambda kc=kc, vc=vc: ops.attention_decode(q, kc, vc, out, None, b, positions, seq_of, table, hq, hkv, hd,
                                                         page, None, 1.0 / math.sqrt(hd), splits, scratch, tickets)
               for kc, vc in caches]
    us = _time(fns, args.iters)
    print(f"attention_decode{' (merge through scratch)' if args.scratch_merge else ''}{' (balanced)' if args.balanced else ''}{' ragged' if args.ragged else ''} batch={b} context={ctx} heads={hq}/{hkv} hd={hd} page={page} splits={splits}: "
          f"{us:.2f} us, {kv_bytes / us / 1e3:.0f} GB/s of cache")


def attention_prefill(args) -> None:
    t, hq, hkv, hd, page = args.tokens, args.q_heads, args.kv_heads, args.head_dim, args.page
    g = torch.Generator(device=DEV).manual_seed(0)
    n_pages = -(-t // page)
    kc = torch.randn(n_pages, hkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    vc = torch.randn(n_pages, hkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    table = torch.randperm(n_pages, device=DEV, generator=g).int().view(1, n_pages)
    q = torch.randn(t, hq * hd, device=DEV, generator=g).to(torch.bfloat16)
    out = torch.empty_like(q)
    tiles = list(range(0, t, ops.PREFILL_TILE_ROWS))[::-1]
    tile_seq = torch.zeros(len(tiles), dtype=torch.int32, device=DEV)
    tile_row0 = torch.tensor(tiles, dtype=torch.int32, device=DEV)
    cu_q = torch.tensor([0, t], dtype=torch.int32, device=DEV)
    kv_len = torch.tensor([t], dtype=torch.int32, device=DEV)
    fn = lambda: ops.attention_prefill(q, kc, vc, out, tile_seq, tile_row0, len(tiles), cu_q, kv_len, table, hq, hkv,
                                       hd, page, None, 1.0 / math.sqrt(hd), kernel=args.kernel)
    us = _time([fn], args.iters)
    ops.check_device_errors()
    flops = 4.0 * hq * hd * t * (t + 1) / 2
    print(f"attention_prefill tokens={t} heads={hq}/{hkv} hd={hd} kernel={args.kernel or 'default'}: {us:.1f} us, "
          f"{flops / us / 1e6:.0f} TFLOP/s (causal)")


def decode_step(args) -> None:
    """One decode step of the whole model as the engine runs it (a replayed graph with arg-max and token
    feedback on the device), optionally with one kind of kernel left out: the difference is what that
    kind costs inside the chain of dependent launches.  With --without the results are WRONG (the
    kernel's output is whatever was in its buffer); only the time means something."""
    from ..config import config_from_dict, preset
    from ..engine import ModelRunner, StepEntry
    from ..weights import tensor_plan
    raw = dict(preset(args.shape))
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    config = config_from_dict(raw)
    g = torch.Generator(device=DEV).manual_seed(0)
    weights = {p.name: (torch.ones(p.shape, dtype=torch.bfloat16, device=DEV) if p.init == "ones" else
                        (torch.randn(p.shape, generator=g, device=DEV, dtype=torch.float32) * 0.02).to(torch.bfloat16))
               for p in tensor_plan(config)}
    batch, ctx_len, page = args.batch, args.context, 16
    cpu = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, raw["vocab_size"], (ctx_len,), generator=cpu).tolist() for _ in range(batch)]
    runner = ModelRunner(config, weights, dtype="bfloat16", page_size=page, num_pages=batch * (ctx_len // page + 8) + 8 + args.iters,
                         max_requests=batch, max_tokens_per_request=ctx_len + 64 + args.iters)
    last = [int(torch.argmax(runner.step([StepEntry(r, toks, [ctx_len - 1])])[0])) for r, toks in enumerate(prompts)]
    keep = {name: getattr(ops, name) for name in ("attention_decode", "attention_decode_balanced", "gemv_qkv_rope",
                                                  "gemv_ksplit", "gemv_bf16", "gemv_norm_bf16")}
    nothing = lambda *a, **k: None
    if args.without == "attention":
        ops.attention_decode = ops.attention_decode_balanced = nothing
    elif args.without == "qkv":
        ops.gemv_qkv_rope = nothing
    elif args.without == "down":
        ops.gemv_ksplit = nothing
    elif args.without in ("gate_up", "output", "vocabulary"):
        def some(x, w, out, mode, *a, **k):
            if (args.without == "gate_up" and mode == ops.SWIGLU_BF16) or (args.without == "output" and mode == ops.ADD_F32):
                return
            keep["gemv_bf16"](x, w, out, mode, *a, **k)

        def some_norm(h, gain, eps, rows, w, out, mode, *a, **k):
            if (args.without == "gate_up" and mode == ops.SWIGLU_BF16) or (args.without == "vocabulary" and mode == ops.STORE_F32):
                return
            keep["gemv_norm_bf16"](h, gain, eps, rows, w, out, mode, *a, **k)
        ops.gemv_bf16, ops.gemv_norm_bf16 = some, some_norm
    toks = runner.greedy_decode_on_device(list(range(batch)), last, 4)           # captures the step
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    runner.greedy_decode_on_device(list(range(batch)), toks[-1].tolist(), args.iters)
    b.record()
    torch.cuda.synchronize()
    for name, fn in keep.items():
        setattr(ops, name, fn)
    ops.check_device_errors()
    print(f"decode step, batch {batch}, context {ctx_len}, {raw['num_hidden_layers']} layers of {args.shape}"
          f"{', WITHOUT ' + args.without + ' (time only)' if args.without else ''}: {a.elapsed_time(b) / args.iters:.4f} ms")


def decode_fused(args) -> None:
    """One decode step of the whole model as ONE persistent kernel (csrc/decode_fused.cu) against the
    same step as the chain of per-part kernels, and where the fused kernel's time goes: block 0 stamps
    the time at every phase boundary."""
    from ..config import config_from_dict, preset
    from ..engine import ModelRunner, StepEntry
    from ..weights import tensor_plan
    raw = dict(preset(args.shape))
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    config = config_from_dict(raw)
    g = torch.Generator(device=DEV).manual_seed(0)
    weights = {p.name: (torch.ones(p.shape, dtype=torch.bfloat16, device=DEV) if p.init == "ones" else
                        (torch.randn(p.shape, generator=g, device=DEV, dtype=torch.float32) * 0.02).to(torch.bfloat16))
               for p in tensor_plan(config)}
    batch, ctx_len, page = args.batch, args.context, 16
    cpu = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, raw["vocab_size"], (ctx_len,), generator=cpu).tolist() for _ in range(batch)]
    results = {}
    for fused in (False, True):
        runner = ModelRunner(config, weights, dtype="bfloat16", page_size=page, num_pages=batch * (ctx_len // page + 8) + 8,
                             max_requests=batch, max_tokens_per_request=ctx_len + 256, fused_decode=fused)
        last = []
        for r, toks in enumerate(prompts):
            last.append(int(torch.argmax(runner.step([StepEntry(r, toks, [ctx_len - 1])])[0])))
        n = args.iters
        toks = runner.greedy_decode_on_device(list(range(batch)), last, 4)       # captures the step
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        toks = runner.greedy_decode_on_device(list(range(batch)), toks[-1].tolist(), n)
        b.record()
        torch.cuda.synchronize()
        ops.check_device_errors()
        results[fused] = a.elapsed_time(b) / n
        if fused:
            f = runner.model._fused
            stamps = torch.zeros(4096, dtype=torch.int64, device=DEV)
            f.params.trace = stamps.data_ptr()
            runner.use_graphs = False
            runner.step([StepEntry(r, [int(t)], [0]) for r, t in enumerate(toks[-1].tolist())])
            torch.cuda.synchronize()
            f.params.trace = None
            layers = raw["num_hidden_layers"]
            names = ["embedding", "barrier"]
            for _ in range(layers):
                names += ["qkv", "barrier", "attention", "barrier", "output", "barrier", "gate/up", "barrier", "down", "barrier"]
            names += ["vocabulary"]
            t = stamps.cpu().tolist()[:len(names)]
            total = {}
            for i in range(1, len(names)):
                total.setdefault(names[i], []).append((t[i] - t[i - 1]) / 1e3)
            print(f"fused kernel, one step seen by block 0: {(t[-1] - t[0]) / 1e3:.0f} us")
            for k, v in total.items():
                print(f"  {k:10s} {len(v):3d} x {sum(v) / len(v):7.2f} us = {sum(v):8.1f} us")
        del runner
        torch.cuda.empty_cache()
    print(f"decode step, batch {batch}, context {ctx_len}, {raw['num_hidden_layers']} layers of {args.shape}: "
          f"chain of kernels {results[False]:.3f} ms, fused kernel {results[True]:.3f} ms")


def main() -> None:
    ops.require_cuda()
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="case", required=True)
    p = sub.add_parser("gemv")
    p.add_argument("--m", type=int, default=8)
    p.add_argument("--n", type=int, default=16384)
    p.add_argument("--k", type=int, default=2048)
    p.add_argument("--mode", default="bf16", choices=["bf16", "f32", "add", "swiglu"])
    p.add_argument("--norm", action="store_true")
    p.add_argument("--ksplit", action="store_true", help="the cluster split-K kernel (gemv_ksplit.cu) instead of gemv_bf16.cu")
    p.add_argument("--prepared", action="store_true", help="the reader of a norm handed over by the kernel before (bfloat16 input + partial sums)")
    p.add_argument("--parts", type=int, default=256, help="--prepared: partial sums per row")
    p.set_defaults(fn=gemv)
    p = sub.add_parser("sample")
    p.add_argument("--rows", type=int, default=8)
    p.add_argument("--vocab", type=int, default=128256)
    p.add_argument("--temperature", type=float, default=0.8)
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--one-block", action="store_true")
    p.set_defaults(fn=sample)
    p = sub.add_parser("add_rmsnorm")
    p.add_argument("--rows", type=int, default=2048)
    p.add_argument("--width", type=int, default=2048)
    p.add_argument("--copies", type=int, default=1)
    p.set_defaults(fn=add_rmsnorm)
    p = sub.add_parser("gemm")
    p.add_argument("--m", type=int, default=2048)
    p.add_argument("--n", type=int, default=16384)
    p.add_argument("--k", type=int, default=2048)
    p.add_argument("--mode", default="bf16", choices=["bf16", "f32", "add", "swiglu"])
    p.add_argument("--kernel", default=None, choices=["single", "pair"])
    p.add_argument("--accumulators", type=int, default=2)
    p.add_argument("--tile-n", type=int, default=0, help="pair kernel: 128, 192 or 256 columns per tile (0: by size)")
    p.set_defaults(fn=gemm)
    p = sub.add_parser("gemm_swap")
    p.add_argument("--m", type=int, default=64)
    p.add_argument("--n", type=int, default=16384)
    p.add_argument("--k", type=int, default=2048)
    p.add_argument("--mode", default="bf16", choices=["bf16", "f32", "add", "swiglu"])
    p.add_argument("--milestones", action="store_true", help="also print block 0's timeline of one launch")
    p.set_defaults(fn=gemm_swap)
    p = sub.add_parser("decode_step")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=2048)
    p.add_argument("--shape", default="llama-3.2-1b")
    p.add_argument("--layers", type=int, default=0)
    p.add_argument("--without", default="", choices=["", "attention", "qkv", "output", "gate_up", "down", "vocabulary"],
                   help="leave one kind of kernel out of the step (wrong results; what it costs inside the chain)")
    p.set_defaults(fn=decode_step)
    p = sub.add_parser("decode_fused")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=2048)
    p.add_argument("--shape", default="llama-3.2-1b")
    p.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has")
    p.set_defaults(fn=decode_fused)
    for name, fn in (("attention_decode", attention_decode), ("attention_prefill", attention_prefill)):
        p = sub.add_parser(name)
        p.add_argument("--batch", type=int, default=8)
        p.add_argument("--context", type=int, default=3072)
        p.add_argument("--tokens", type=int, default=2048)
        p.add_argument("--q-heads", type=int, default=32)
        p.add_argument("--kv-heads", type=int, default=8)
        p.add_argument("--head-dim", type=int, default=64)
        p.add_argument("--page", type=int, default=16)
        p.add_argument("--splits", type=int, default=0)
        p.add_argument("--kernel", default=None, choices=["tc", "mma"], help="prefill: insist on one kernel")
        p.add_argument("--copies", type=int, default=0, help="decode: cache copies used in turn (default: enough to exceed L2; 1: the cache stays in L2)")
        p.add_argument("--balanced", action="store_true", help="decode: the kernel that deals the keys evenly over a fixed grid")
        p.add_argument("--ragged", action="store_true", help="decode: contexts from a quarter of --context up to it")
        p.add_argument("--scratch-merge", action="store_true",
                       help="decode: merge the splits through global scratch and tickets, not inside a cluster")
        p.set_defaults(fn=fn)
    for sp in sub.choices.values():
        sp.add_argument("--iters", type=int, default=200)
    args = ap.parse_args()
    args.fn(args)


if __name__ == "__main__":
    main()
