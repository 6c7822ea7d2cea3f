"""Each part alone against its plain formula, and the generality of the assembly: a toy mixer
with state of its own, a toy routed feed-forward and another position encoding are defined
HERE, registered, built into a model with a schedule that repeats a layer and shares a cache,
and stepped through the engine - without a change to the package's files.

The toy parts are written with torch ops (they are test code, not product kernels); the model
they form is no published architecture.
"""
import math

import pytest
import torch

import plain_llama as plain
import replay_util as ru
from helpers import random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# ---------------------------------------------------------------------------------------------
# parts alone
# ---------------------------------------------------------------------------------------------
def _runtime(dtype, page=8):
    from nanoinfer_b200.engine.runtime import Runtime, parse_dtype
    return Runtime(device=torch.device(DEV), dtype=parse_dtype(dtype), page_size=page)


def _close(got, want, dtype):
    """float32: rounding in another order.  bfloat16: a part chains two or three products whose
    operands are rounded to 8 bits of mantissa (2^-9 relative each): the error is bounded
    against the size of the part's output, 2 % of its largest value."""
    if dtype == "float32":
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
    else:
        err = (got - want).abs().max().item()
        assert err <= 0.02 * want.abs().max().item(), f"max error {err:.4g} vs scale {want.abs().max().item():.4g}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(dtype):
    from nanoinfer_b200.config import NormSpec, part
    rt = _runtime(dtype)
    d = 120
    g = torch.Generator().manual_seed(0)
    gain = torch.randn(d, generator=g) * 0.1 + 1.0
    norm = part("norm", "rmsnorm")(NormSpec("rmsnorm", 1e-6), d, {"weight": gain.to(torch.bfloat16)}, rt)
    h = torch.randn(7, d, generator=g).to(DEV)
    delta = torch.randn(7, d, generator=g).to(rt.dtype).to(DEV)
    want_h = h.cpu() + delta.cpu().float()
    x = norm.forward(h, delta)
    assert x.dtype == rt.dtype
    torch.testing.assert_close(h.cpu(), want_h)
    _close(x.cpu().float(), plain.rms_norm(want_h, gain.to(torch.bfloat16), 1e-6), dtype)


def test_rotary_part_constants():
    from nanoinfer_b200.config import PositionSpec, RopeScaling, part
    rt = _runtime("float32")
    sc = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
              original_max_position_embeddings=256)
    enc = part("position", "rope")(PositionSpec("rope", 10000.0, 48, "interleaved", RopeScaling(**sc)), 0, {}, rt)
    torch.testing.assert_close(enc.inv_freq.cpu(), plain.rope_inv_freq(48, 10000.0, sc), rtol=3e-7, atol=0)
    assert enc.interleaved and enc.rotary_dim == 48
    none = part("position", "none")(PositionSpec("none"), 0, {}, rt)
    assert none.rotary_dim == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu_part(dtype):
    from nanoinfer_b200.config import FeedForwardSpec, part
    rt = _runtime(dtype)
    d, inter = 96, 200
    g = torch.Generator().manual_seed(1)
    w = {k: (torch.randn(s, generator=g) * 0.05).to(torch.bfloat16)
         for k, s in (("gate", (inter, d)), ("up", (inter, d)), ("down", (d, inter)))}
    ffn = part("feed_forward", "swiglu")(FeedForwardSpec("swiglu", inter), d, w, rt)
    for rows in (3, 40):          # the skinny kernel and the library product
        x = torch.randn(rows, d, generator=g).to(rt.dtype)
        y = ffn.forward(x.to(DEV), None)
        want = plain.swiglu_ffn(x.float(), w["gate"], w["up"], w["down"])
        _close(y.cpu().float(), want, dtype)
        if dtype == "bfloat16" and rows <= 16:
            h = torch.randn(rows, d, generator=g).to(DEV)
            h0 = h.clone()
            assert ffn.forward(x.to(DEV), None, residual=h) is None      # fused epilogue
            _close((h - h0).cpu(), want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,pairing,hd", [(None, "half", 64), (9, "interleaved", 32), (None, "half", 16)])
def test_attention_part_and_block(dtype, window, pairing, hd):
    """PagedAttention alone (two steps: a portion, then the rest token by token) and inside a
    PreNormBlock, against the plain attention block."""
    from nanoinfer_b200.cache import CacheManager, GroupSpec
    from nanoinfer_b200.config import FeedForwardSpec, LayerSpec, MixerSpec, NormSpec, PositionSpec, part
    from nanoinfer_b200.engine.step import CacheView, StepContext
    rt = _runtime(dtype, page=8)
    d, n_q, n_kv = 80, 4, 2
    g = torch.Generator().manual_seed(hd)
    pos_spec = PositionSpec("rope", 10000.0, hd, pairing, None)
    spec = MixerSpec("attention", n_q, n_kv, hd, window, 1.0 / math.sqrt(hd), pos_spec)
    names = {"q": (n_q * hd, d), "k": (n_kv * hd, d), "v": (n_kv * hd, d), "o": (d, n_q * hd)}
    w = {k: (torch.randn(s, generator=g) * 0.08).to(torch.bfloat16) for k, s in names.items()}
    mixer = part("mixer", "attention")(spec, d, w, rt)
    need = mixer.cache_need()
    assert (need.num_kv_heads, need.head_dim, need.window) == (n_kv, hd, window)

    T = 29
    x = torch.randn(T, d, generator=g).to(rt.dtype)
    pw = {f"p.{k}_proj.weight": v for k, v in w.items()}
    want = plain.attention_block(x.float(), pw, "p", n_q, n_kv, hd, torch.arange(T),
                                 plain.rope_inv_freq(hd, 10000.0, None), pairing, spec.softmax_scale, window)

    cm = CacheManager([GroupSpec(n_kv, hd, window)], [8], 8, 2, 64)
    slot = cm.admit("r")
    shape = (8, n_kv, 8, hd)
    cache = CacheView(group=0, pages={"k": torch.zeros(shape, dtype=rt.dtype, device=DEV),
                                      "v": torch.zeros(shape, dtype=rt.dtype, device=DEV)})

    def ctx_for(start, n):
        from nanoinfer_b200.engine.step import upload_plans
        cm.append("r", n)
        i32 = dict(dtype=torch.int32, device=DEV)
        width = cm.table_width
        return StepContext(
            n_tokens=n, n_seqs=1, n_logit_rows=0, tokens=torch.zeros(n, **i32),
            positions=torch.arange(start, start + n, **i32), seq_of_token=torch.zeros(n, **i32),
            cu_q=torch.tensor([0, n], **i32), kv_len=torch.tensor([start + n], **i32),
            slots=torch.tensor([slot], **i32), logit_rows=torch.zeros(0, **i32),
            block_tables=[torch.from_numpy(cm.table_rows(0, [slot], width)).to(DEV)],
            host_q_lens=[n], host_kv_lens=[start + n], host_slots=[slot], max_q_len=n, max_kv_len=start + n,
            decode_only=(n == 1), plans=upload_plans([mixer], [n], [start], DEV))   # the mixer's own tiling of the step

    outs = [mixer.forward(x[:20].to(DEV), ctx_for(0, 20), cache)]
    for t in range(20, T):
        outs.append(mixer.forward(x[t:t + 1].to(DEV), ctx_for(t, 1), cache))
    got = torch.cat(outs).cpu().float()
    _close(got, want, dtype)

    # the same mixer inside a block with norms and a feed-forward
    inter = 120
    fw = {k: (torch.randn(s, generator=g) * 0.05).to(torch.bfloat16)
          for k, s in (("gate", (inter, d)), ("up", (inter, d)), ("down", (d, inter)))}
    gains = {"weight": torch.ones(d, dtype=torch.bfloat16)}
    layer = LayerSpec(spec, FeedForwardSpec("swiglu", inter), NormSpec("rmsnorm", 1e-5), NormSpec("rmsnorm", 1e-5))
    weights_of = {"mixer": w, "feed_forward": fw, "mixer_norm": gains, "ffn_norm": gains}
    block = part("arrangement", "pre_norm")(layer, d, lambda what: weights_of[what], rt)
    cm.free("r")
    slot = cm.admit("r")
    h0 = torch.randn(T, d, generator=g)
    h = h0.clone().to(DEV)
    delta = block.forward(h, None, ctx_for(0, T), cache)
    if delta is not None:
        h += delta.float()
    a = h0 + plain.attention_block(plain.rms_norm(h0, gains["weight"], 1e-5), pw, "p", n_q, n_kv, hd, torch.arange(T),
                                   plain.rope_inv_freq(hd, 10000.0, None), pairing, spec.softmax_scale, window)
    want_h = a + plain.swiglu_ffn(plain.rms_norm(a, gains["weight"], 1e-5), fw["gate"], fw["up"], fw["down"])
    _close(h.cpu(), want_h, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,hd,n_q,n_kv", [(None, 32, 4, 2), (7, 48, 3, 1)])
def test_a_position_encoding_that_biases_the_scores(dtype, window, hd, n_q, n_kv):
    """Another kind of position encoding, defined and registered here: nothing is rotated; head h
    adds -BIAS_BASE^-(h+1) * (query position - key position) to its scaled scores.  The mixer
    reads the slopes from its encoding and hands them to the attention kernel; a portion and
    single tokens give what the whole sequence gives.  The slope of head 0 is made large, so
    that each of its rows is the value of its own position: a bias that was dropped, or had the
    wrong sign, would average the values instead."""
    from nanoinfer_b200.cache import CacheManager, GroupSpec
    from nanoinfer_b200.config import MixerSpec, PositionSpec, part, register_part
    from nanoinfer_b200.engine.step import CacheView, StepContext, upload_plans
    from nanoinfer_b200.parts.position import NoEncoding
    BIAS_BASE, STEEP = 2.0, 40.0

    class LinearScoreBias(NoEncoding):
        def __init__(self, spec, hidden_size, weights, rt):
            super().__init__(spec, hidden_size, weights, rt)
            slopes = [STEEP] + [BIAS_BASE ** -(h + 1) for h in range(1, n_q)]
            self.head_slopes = torch.tensor(slopes, dtype=torch.float32, device=rt.device)

    register_part("position", "toy_linear_score_bias", LinearScoreBias, replace=True)
    rt = _runtime(dtype, page=8)
    d, T, cut = 72, 41, 26
    g = torch.Generator().manual_seed(hd)
    spec = MixerSpec("attention", n_q, n_kv, hd, window, 1.0 / math.sqrt(hd),
                     PositionSpec("toy_linear_score_bias", 10000.0, 0, "half", None))
    names = {"q": (n_q * hd, d), "k": (n_kv * hd, d), "v": (n_kv * hd, d), "o": (d, n_q * hd)}
    w = {k: (torch.randn(s, generator=g) * 0.1).to(torch.bfloat16) for k, s in names.items()}
    mixer = part("mixer", "attention")(spec, d, w, rt)
    x = torch.randn(T, d, generator=g).to(rt.dtype)

    # plain: the same projections, scores with the bias, whole sequence
    with plain.precision(torch.float32):
        xf = x.float()
        q = (xf @ w["q"].float().t()).view(T, n_q, hd)
        k = (xf @ w["k"].float().t()).view(T, n_kv, hd)
        v = (xf @ w["v"].float().t()).view(T, n_kv, hd)
        i = torch.arange(T)
        mask = i[None, :] <= i[:, None]
        if window is not None:
            mask &= i[None, :] > i[:, None] - window
        att = torch.empty(T, n_q, hd)
        slopes = mixer.position.head_slopes.cpu()
        for h in range(n_q):
            kh, vh = k[:, h // (n_q // n_kv)], v[:, h // (n_q // n_kv)]
            sc = (q[:, h] @ kh.t()) * spec.softmax_scale + slopes[h] * (i[None, :] - i[:, None]).float()
            att[:, h] = torch.softmax(sc.masked_fill(~mask, float("-inf")), dim=-1) @ vh
        want = att.reshape(T, n_q * hd) @ w["o"].float().t()
        assert torch.allclose(att[:, 0], v[:, 0], atol=1e-6)          # the steep head sees itself alone

    cm = CacheManager([GroupSpec(n_kv, hd, window)], [8], 8, 2, 64)
    slot = cm.admit("r")
    shape = (8, n_kv, 8, hd)
    cache = CacheView(group=0, pages={"k": torch.zeros(shape, dtype=rt.dtype, device=DEV),
                                      "v": torch.zeros(shape, dtype=rt.dtype, device=DEV)})

    def ctx_for(start, n):
        cm.append("r", n)
        i32 = dict(dtype=torch.int32, device=DEV)
        return StepContext(
            n_tokens=n, n_seqs=1, n_logit_rows=0, tokens=torch.zeros(n, **i32),
            positions=torch.arange(start, start + n, **i32), seq_of_token=torch.zeros(n, **i32),
            cu_q=torch.tensor([0, n], **i32), kv_len=torch.tensor([start + n], **i32),
            slots=torch.tensor([slot], **i32), logit_rows=torch.zeros(0, **i32),
            block_tables=[torch.from_numpy(cm.table_rows(0, [slot], cm.table_width)).to(DEV)],
            host_q_lens=[n], host_kv_lens=[start + n], host_slots=[slot], max_q_len=n, max_kv_len=start + n,
            decode_only=(n == 1), plans=upload_plans([mixer], [n], [start], DEV))

    outs = [mixer.forward(x[:cut].to(DEV), ctx_for(0, cut), cache)]
    for t in range(cut, T):
        outs.append(mixer.forward(x[t:t + 1].to(DEV), ctx_for(t, 1), cache))
    _close(torch.cat(outs).cpu().float(), want, dtype)


# ---------------------------------------------------------------------------------------------
# toy parts, defined in the test
# ---------------------------------------------------------------------------------------------
# A routed part takes a discrete decision.  Where the plain router's best two experts are closer
# than this share of the largest router logit, bfloat16 rounding may pick the other one, and
# everything after that position differs for good reason: bfloat16 runs are compared up to the
# first such position of a request (float32 runs are compared everywhere).
CLOSE_CALL = 0.05
DECAY = 0.9
STATE = 24
EXPERTS, EXPERT_WIDTH = 3, 40
ROPE_DIVISOR = 4.0


def _register_toys():
    from nanoinfer_b200.config import (FeedForwardSpec, LayerRun, LayerSpec, MixerSpec, ModelConfig, NormSpec,
                                       PositionSpec, register_architecture, register_part)
    from nanoinfer_b200.parts.base import Part, StateNeed, WeightSlot
    from nanoinfer_b200.parts.position import RotaryEncoding

    class RunningStateMixer(Part):
        """s_t = DECAY * s_{t-1} + W_in x_t ;  y_t = W_out s_t.  One FP32 state vector per request."""

        @staticmethod
        def weight_slots(spec, hidden_size):
            return {"w_in": WeightSlot((STATE, hidden_size)), "w_out": WeightSlot((hidden_size, STATE))}

        def __init__(self, spec, hidden_size, weights, rt):
            super().__init__(spec, hidden_size, weights, rt)
            self.w_in = weights["w_in"].to(rt.device, torch.float32)
            self.w_out = weights["w_out"].to(rt.device, torch.float32)

        def cache_need(self):
            return StateNeed((STATE,), "float32")

        def forward(self, x, ctx, cache):
            u = x.float() @ self.w_in.t()
            y = torch.empty(x.shape[0], self.hidden_size, dtype=torch.float32, device=x.device)
            at = 0
            for n, slot in zip(ctx.host_q_lens, ctx.host_slots):   # tokens of a request in order
                s = cache.state[slot]
                for t in range(at, at + n):
                    s = DECAY * s + u[t]
                    y[t] = self.w_out @ s
                cache.state[slot] = s
                at += n
            return y.to(self.rt.dtype)

    class Top1Experts(Part):
        """Router logits in FP32, the best expert alone: y = W2[e] relu(W1[e] x)."""

        @staticmethod
        def weight_slots(spec, hidden_size):
            return {"router": WeightSlot((EXPERTS, hidden_size)),
                    "w1": WeightSlot((EXPERTS, EXPERT_WIDTH, hidden_size)),
                    "w2": WeightSlot((EXPERTS, hidden_size, EXPERT_WIDTH))}

        def __init__(self, spec, hidden_size, weights, rt):
            super().__init__(spec, hidden_size, weights, rt)
            self.w = {k: v.to(rt.device, torch.float32) for k, v in weights.items()}

        def forward(self, x, ctx):
            xf = x.float()
            e = torch.argmax(xf @ self.w["router"].t(), dim=-1)
            hid = torch.relu(torch.einsum("tfd,td->tf", self.w["w1"][e], xf))
            return torch.einsum("tdf,tf->td", self.w["w2"][e], hid).to(self.rt.dtype)

    class SlowRope(RotaryEncoding):
        """Rotary encoding with every frequency divided by ROPE_DIVISOR."""

        def __init__(self, spec, hidden_size, weights, rt):
            super().__init__(spec, hidden_size, weights, rt)
            self.inv_freq = self.inv_freq / ROPE_DIVISOR

    register_part("mixer", "toy_running_state", RunningStateMixer, replace=True)
    register_part("feed_forward", "toy_top1_experts", Top1Experts, replace=True)
    register_part("position", "toy_slow_rope", SlowRope, replace=True)

    def parse(raw):
        d, hd = raw["width"], raw["head"]
        norm = NormSpec("rmsnorm", raw["eps"])

        def att(window, pos_kind):
            return MixerSpec("attention", raw["heads"], raw["kv_heads"], hd, window, 1.0 / math.sqrt(hd),
                             PositionSpec(pos_kind, 10000.0, hd if pos_kind != "none" else 0, "half", None))
        layers = (
            LayerSpec(att(None, "toy_slow_rope"), FeedForwardSpec("swiglu", raw["ffn"]), norm, norm),
            LayerSpec(MixerSpec("toy_running_state"), FeedForwardSpec("toy_top1_experts"), norm, norm),
            LayerSpec(att(raw["window"], "none"), FeedForwardSpec("swiglu", raw["ffn"]), norm, norm),
        )
        # layer 0 runs twice (own cache each time); the last run reads run 2's pages
        schedule = (LayerRun(0), LayerRun(1), LayerRun(2), LayerRun(0), LayerRun(2, cache_of=2))
        return ModelConfig("ToyHybridForTest", d, raw["vocab"], raw["max_pos"], layers, schedule, norm,
                           tie_word_embeddings=True)

    def name(scope, slot):
        return "toy." + ".".join(str(s) for s in scope) + "." + slot

    register_architecture("ToyHybridForTest", parse, name, replace=True)


TOY_RAW = {"architectures": ["ToyHybridForTest"], "width": 64, "head": 16, "heads": 4, "kv_heads": 2, "ffn": 96,
           "vocab": 200, "max_pos": 256, "eps": 1e-5, "window": 11}


def _toy_plain(w, tokens):
    """The toy model, whole sequence, from the formulas above and plain_llama's parts.
    Returns (logits, first position whose expert choice is a close call or None)."""
    raw = TOY_RAW
    d, hd, nq, nkv = raw["width"], raw["head"], raw["heads"], raw["kv_heads"]
    T = len(tokens)
    pos = torch.arange(T)
    scale = 1.0 / math.sqrt(hd)
    slow = plain.rope_inv_freq(hd, 10000.0, None) / ROPE_DIVISOR
    W = {k: v.float() for k, v in w.items()}

    def norm(h, key):
        return plain.rms_norm(h, W[key], raw["eps"])

    def att(h, i, inv_freq, window, kv_from=None):
        x = norm(h, f"toy.layer.{i}.mixer_norm.weight")
        q = (x @ W[f"toy.layer.{i}.mixer.q"].t()).view(T, nq, hd)
        k = (x @ W[f"toy.layer.{i}.mixer.k"].t()).view(T, nkv, hd)
        v = (x @ W[f"toy.layer.{i}.mixer.v"].t()).view(T, nkv, hd)
        if inv_freq is not None:
            q, k = plain.rope(q, pos, inv_freq, "half"), plain.rope(k, pos, inv_freq, "half")
        if kv_from is not None:
            k, v = kv_from
        o = plain.attention(q, k, v, scale, window).reshape(T, nq * hd)
        return h + o @ W[f"toy.layer.{i}.mixer.o"].t(), (k, v)

    def swiglu(h, i):
        x = norm(h, f"toy.layer.{i}.ffn_norm.weight")
        p = f"toy.layer.{i}.feed_forward"
        return h + plain.swiglu_ffn(x, W[f"{p}.gate"], W[f"{p}.up"], W[f"{p}.down"])

    h = plain.embedding(W["toy.embedding.weight"], torch.tensor(tokens))
    h, _ = att(h, 0, slow, None)
    h = swiglu(h, 0)
    # layer 1: running state + routed experts
    x = norm(h, "toy.layer.1.mixer_norm.weight")
    u = x @ W["toy.layer.1.mixer.w_in"].t()
    s = torch.zeros(STATE)
    y = torch.empty(T, d)
    for t in range(T):
        s = DECAY * s + u[t]
        y[t] = W["toy.layer.1.mixer.w_out"] @ s
    h = h + y
    x = norm(h, "toy.layer.1.ffn_norm.weight")
    router = x @ W["toy.layer.1.feed_forward.router"].t()
    e = torch.argmax(router, dim=-1)
    top2 = torch.topk(router, 2, dim=-1).values
    close = torch.nonzero((top2[:, 0] - top2[:, 1]) < CLOSE_CALL * router.abs().max())
    first_close = int(close[0]) if close.numel() else None
    hid = torch.relu(torch.einsum("tfd,td->tf", W["toy.layer.1.feed_forward.w1"][e], x))
    h = h + torch.einsum("tdf,tf->td", W["toy.layer.1.feed_forward.w2"][e], hid)
    h, kv2 = att(h, 2, None, TOY_RAW["window"])
    h = swiglu(h, 2)
    h, _ = att(h, 0, slow, None)
    h = swiglu(h, 0)
    h, _ = att(h, 2, None, TOY_RAW["window"], kv_from=kv2)
    h = swiglu(h, 2)
    return norm(h, "toy.final_norm.weight") @ W["toy.embedding.weight"].t(), first_close


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_parts_register_build_and_step(tmp_path, dtype):
    from nanoinfer_b200.config import load_config
    from nanoinfer_b200.engine import ModelRunner
    from nanoinfer_b200.weights import load_weights, write_random_model
    _register_toys()
    d = str(tmp_path / "toy")
    write_random_model(d, TOY_RAW, seed=5, std=0.08)        # random-weights mode knows the toy tensors
    cfg = load_config(d)
    weights = load_weights(d, cfg)
    assert "toy.layer.1.mixer.w_in" in weights and "toy.layer.1.feed_forward.router" in weights
    # token seeds chosen so that the plain router has no close call in these requests
    reqs = {f"t{i}": random_tokens(TOY_RAW["vocab"], n, seed)
            for i, (n, seed) in enumerate([(9, 40), (70, 75), (31, 41), (120, 100)])}
    plain_out = {rid: _toy_plain(weights, toks) for rid, toks in reqs.items()}
    want = {rid: o[0] for rid, o in plain_out.items()}
    limit = {rid: (len(reqs[rid]) if o[1] is None or dtype == "float32" else o[1]) for rid, o in plain_out.items()}
    assert sum(limit.values()) >= 0.9 * sum(len(t) for t in reqs.values()), "too little left to compare"
    for cut in (ru.whole, ru.ragged, ru.mixed):
        steps = cut(reqs)
        runner = ModelRunner(cfg, weights, dtype=dtype, page_size=8,
                             num_pages=ru.max_live_tokens(steps, 64) // 8, max_requests=4)
        # three needs, three kinds of cache: all keys, a window of keys, a state slot
        assert [g.window for g in runner.cache.groups] == [None, TOY_RAW["window"]]
        assert len(runner._state_runs) == 1 and runner.caches[4].writable is False
        assert not runner.decode_graphs_ok          # the host-side toy mixer declares no graph safety
        got = ru.run_trace(runner, steps)
        assert len(got) == sum(len(t) for t in reqs.values())
        got = {k: v for k, v in got.items() if k[1] < limit[k[0]]}
        ru.compare(got, want, dtype, label=f"toy/{cut.__name__}/{dtype}")
        runner.cache.check_consistency()
        assert all(p.num_free == p.num_pages for p in runner.cache.pools)


# ---------------------------------------------------------------------------------------------
# more toy parts: a plan of the part's own, state under captured graphs, a cache that is not K/V
# ---------------------------------------------------------------------------------------------
LATENT = 12


def _register_more_toys():
    import numpy as np
    from nanoinfer_b200.config import (EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerRun, LayerSpec, MixerSpec,
                                       ModelConfig, NormSpec, PositionSpec, register_architecture, register_part)
    from nanoinfer_b200.parts.base import PagedNeed, Part, StateNeed, StepPlan, WeightSlot
    from nanoinfer_b200.parts.embedding import TableEmbedding
    from nanoinfer_b200.parts.head import LinearHead

    class ShiftMixer(Part):
        """y_t = W1 x_t + W2 x_{t-1} (x_{-1} = 0).  The token before a portion's first token comes
        from the request's state slot.  The part plans its own work: per request, the index of its
        first and of its last token in the step.  Nothing is decided on the host in forward, so any
        step may be captured and replayed."""
        graph_safe = "all"

        @staticmethod
        def weight_slots(spec, hidden_size):
            return {"w1": WeightSlot((hidden_size, hidden_size)), "w2": WeightSlot((hidden_size, hidden_size))}

        def __init__(self, spec, hidden_size, weights, rt):
            super().__init__(spec, hidden_size, weights, rt)
            self.w1 = weights["w1"].to(rt.device, torch.float32)
            self.w2 = weights["w2"].to(rt.device, torch.float32)

        def cache_need(self):
            return StateNeed((self.hidden_size,), "float32")

        @staticmethod
        def plan_step(q_lens, starts):
            ends = np.cumsum(q_lens)
            return StepPlan({"first_token": (ends - np.asarray(q_lens)).astype(np.int32),
                             "last_token": (ends - 1).astype(np.int32)}, {"n_requests": len(q_lens)})

        def forward(self, x, ctx, cache):
            plan = ctx.plan_of(self)
            assert plan.scalars["n_requests"] == ctx.n_seqs
            xf = x.float()
            slots = ctx.slots.long()
            prev = torch.roll(xf, 1, 0)
            prev.index_copy_(0, plan.arrays["first_token"].long(), cache.state.index_select(0, slots))
            cache.state.index_copy_(0, slots, xf.index_select(0, plan.arrays["last_token"].long()))
            return (xf @ self.w1.t() + prev @ self.w2.t()).to(self.rt.dtype)

    class DeviceRunningState(Part):
        """s_t = DECAY * s_{t-1} + W_in x_t ; y_t = W_out s_t, with the state update of single-token
        steps done by device-side index operations: such steps may be captured ("decode").  A step
        that ran twice would decay and add twice."""
        graph_safe = "decode"

        @staticmethod
        def weight_slots(spec, hidden_size):
            return {"w_in": WeightSlot((STATE, hidden_size)), "w_out": WeightSlot((hidden_size, STATE))}

        def __init__(self, spec, hidden_size, weights, rt):
            super().__init__(spec, hidden_size, weights, rt)
            self.w_in = weights["w_in"].to(rt.device, torch.float32)
            self.w_out = weights["w_out"].to(rt.device, torch.float32)

        def cache_need(self):
            return StateNeed((STATE,), "float32")

        def forward(self, x, ctx, cache):
            u = x.float() @ self.w_in.t()
            if ctx.decode_only:
                slots = ctx.slots.long()
                s = cache.state.index_select(0, slots) * DECAY + u
                cache.state.index_copy_(0, slots, s)
                return (s @ self.w_out.t()).to(self.rt.dtype)
            y = torch.empty(x.shape[0], self.hidden_size, dtype=torch.float32, device=x.device)
            at = 0
            for n, slot in zip(ctx.host_q_lens, ctx.host_slots):
                s = cache.state[slot]
                for t in range(at, at + n):
                    s = DECAY * s + u[t]
                    y[t] = self.w_out @ s
                cache.state[slot] = s
                at += n
            return y.to(self.rt.dtype)

    class LatentMeanMixer(Part):
        """Keeps ONE small vector per token in pages (a cache that is not keys and values):
        c_t = W_c x_t ; y_t = W_o mean(c_0 .. c_t)."""

        @staticmethod
        def weight_slots(spec, hidden_size):
            return {"w_c": WeightSlot((LATENT, hidden_size)), "w_o": WeightSlot((hidden_size, LATENT))}

        def __init__(self, spec, hidden_size, weights, rt):
            super().__init__(spec, hidden_size, weights, rt)
            self.w_c = weights["w_c"].to(rt.device, torch.float32)
            self.w_o = weights["w_o"].to(rt.device, torch.float32)

        def cache_need(self):
            return PagedNeed((("latent", (LATENT,)),), None)

        def forward(self, x, ctx, cache):
            pages = cache.pages["latent"]                      # [P, page, LATENT]
            page = pages.shape[1]
            c = (x.float() @ self.w_c.t()).to(pages.dtype)
            table = ctx.block_tables[cache.group].cpu()
            y = torch.empty(x.shape[0], self.hidden_size, dtype=torch.float32, device=x.device)
            at = 0
            for i, (n, kv) in enumerate(zip(ctx.host_q_lens, ctx.host_kv_lens)):
                start = kv - n
                for t in range(n):
                    pos = start + t
                    pages[int(table[i, pos // page]), pos % page] = c[at + t]
                held = torch.cat([pages[int(table[i, b])] for b in range(-(-kv // page))])[:kv].float()
                means = held.cumsum(0) / torch.arange(1, kv + 1, device=x.device)[:, None]
                y[at:at + n] = means[start:] @ self.w_o.t()
                at += n
            return y.to(self.rt.dtype)

    class ScaledTable(TableEmbedding):
        """Rows of the table times EMBED_SCALE (a constant of its spec)."""

        def __init__(self, spec, hidden_size, weights, rt):
            super().__init__(spec, hidden_size, weights, rt)
            self.factor = float(spec.extra_dict()["scale"])

        def forward(self, tokens, h):
            super().forward(tokens, h)
            h.mul_(self.factor)

    class SoftCapHead(LinearHead):
        """cap * tanh(logits / cap) over the linear head's logits; here with a matrix of its own
        even when the model's configuration ties the head (its spec is not tied)."""

        def __init__(self, spec, hidden_size, weights, rt):
            super().__init__(spec, hidden_size, weights, rt)
            self.cap = float(spec.extra_dict()["cap"])

        def forward(self, h, delta, norm, ctx):
            logits = super().forward(h, delta, norm, ctx)
            return torch.tanh(logits / self.cap) * self.cap

    register_part("embedding", "toy_scaled_table", ScaledTable, replace=True)
    register_part("head", "toy_soft_cap", SoftCapHead, replace=True)
    register_part("mixer", "toy_shift", ShiftMixer, replace=True)
    register_part("mixer", "toy_device_state", DeviceRunningState, replace=True)
    register_part("mixer", "toy_latent_mean", LatentMeanMixer, replace=True)

    def parse(raw):
        d, hd = raw["width"], raw["head"]
        norm = NormSpec("rmsnorm", raw["eps"])
        ffn = FeedForwardSpec("swiglu", raw["ffn"])

        def att(window):
            return MixerSpec("attention", raw["heads"], raw["kv_heads"], hd, window, 1.0 / math.sqrt(hd),
                             PositionSpec("rope", 10000.0, hd, "half", None))
        kinds = {"shift": MixerSpec("toy_shift"), "state": MixerSpec("toy_device_state"),
                 "latent": MixerSpec("toy_latent_mean"), "attention": att(None), "window": att(raw["window"])}
        layers = tuple(LayerSpec(kinds[k], ffn, norm, norm) for k in raw["mixers"])
        ends = {}
        if raw.get("embed_scale") is not None:
            ends["embedding"] = EmbeddingSpec("toy_scaled_table", extra=(("scale", raw["embed_scale"]),))
        if raw.get("soft_cap") is not None:
            ends["head"] = HeadSpec("toy_soft_cap", extra=(("cap", raw["soft_cap"]),))
        return ModelConfig("ToyMixersForTest", d, raw["vocab"], raw["max_pos"], layers,
                           tuple(LayerRun(i) for i in range(len(layers))), norm, tie_word_embeddings=False, **ends)

    def name(scope, slot):
        return "toy2." + ".".join(str(s) for s in scope) + "." + slot

    register_architecture("ToyMixersForTest", parse, name, replace=True)


def _toy2_raw(mixers):
    return {"architectures": ["ToyMixersForTest"], "width": 64, "head": 16, "heads": 4, "kv_heads": 2, "ffn": 96,
            "vocab": 210, "max_pos": 512, "eps": 1e-5, "window": 20, "mixers": list(mixers)}


def _toy2_plain(raw, w, tokens):
    d, hd, nq, nkv = raw["width"], raw["head"], raw["heads"], raw["kv_heads"]
    T = len(tokens)
    W = {k: v.float() for k, v in w.items()}
    pos = torch.arange(T)
    inv_freq = plain.rope_inv_freq(hd, 10000.0, None)
    h = plain.embedding(W["toy2.embedding.weight"], torch.tensor(tokens)) * (raw.get("embed_scale") or 1.0)
    for i, kind in enumerate(raw["mixers"]):
        p = f"toy2.layer.{i}"
        x = plain.rms_norm(h, W[f"{p}.mixer_norm.weight"], raw["eps"])
        if kind == "shift":
            prev = torch.cat([torch.zeros(1, d), x[:-1]])
            y = x @ W[f"{p}.mixer.w1"].t() + prev @ W[f"{p}.mixer.w2"].t()
        elif kind == "state":
            u = x @ W[f"{p}.mixer.w_in"].t()
            s, y = torch.zeros(STATE), torch.empty(T, d)
            for t in range(T):
                s = DECAY * s + u[t]
                y[t] = W[f"{p}.mixer.w_out"] @ s
        elif kind == "latent":
            c = x @ W[f"{p}.mixer.w_c"].t()
            y = (c.cumsum(0) / torch.arange(1, T + 1)[:, None]) @ W[f"{p}.mixer.w_o"].t()
        else:
            q = plain.rope((x @ W[f"{p}.mixer.q"].t()).view(T, nq, hd), pos, inv_freq, "half")
            k = plain.rope((x @ W[f"{p}.mixer.k"].t()).view(T, nkv, hd), pos, inv_freq, "half")
            v = (x @ W[f"{p}.mixer.v"].t()).view(T, nkv, hd)
            window = raw["window"] if kind == "window" else None
            y = plain.attention(q, k, v, 1.0 / math.sqrt(hd), window).reshape(T, nq * hd) @ W[f"{p}.mixer.o"].t()
        h = h + y
        x = plain.rms_norm(h, W[f"{p}.ffn_norm.weight"], raw["eps"])
        f = f"{p}.feed_forward"
        h = h + plain.swiglu_ffn(x, W[f"{f}.gate"], W[f"{f}.up"], W[f"{f}.down"])
    logits = plain.rms_norm(h, W["toy2.final_norm.weight"], raw["eps"]) @ W["toy2.lm_head.weight"].t()
    cap = raw.get("soft_cap")
    return logits if cap is None else torch.tanh(logits / cap) * cap


def _fixed_portions(requests, size, tail):
    """Portions of one size step after step (they come back, so they are captured), then the last
    ``tail`` tokens one by one; one request at a time."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        cuts = list(range(0, head, size)) + [head] + list(range(head + 1, len(toks)))
        for a, b in zip(cuts, cuts[1:] + [len(toks)]):
            if a < b:
                steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[a:b], "want": list(range(b - a))}],
                              "end": [rid] if b == len(toks) else []})
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mixers,decode_graphs,portion_graphs", [
    (("shift", "attention"), True, True),                 # own plan + state, every step capturable
    (("shift", "state", "window"), True, False),          # a state update that must not run twice; decode steps captured
    (("latent", "attention", "window"), False, False),    # a paged cache that is not K/V; host-side mixer: never captured
])
def test_parts_with_plans_state_and_other_caches(tmp_path, mixers, decode_graphs, portion_graphs, dtype):
    """Parts defined here, with hooks of their own, through the engine's step function, captured
    graphs included, in all cuts - without a change to the package's files."""
    from nanoinfer_b200.config import load_config
    from nanoinfer_b200.engine import ModelRunner
    from nanoinfer_b200.weights import load_weights, write_random_model
    _register_more_toys()
    raw = _toy2_raw(mixers)
    d = str(tmp_path / "toy2")
    write_random_model(d, raw, seed=6, std=0.08)
    cfg = load_config(d)
    weights = load_weights(d, cfg)
    reqs = {f"t{i}": random_tokens(raw["vocab"], n, 300 + i) for i, n in enumerate([9, 70, 31, 120])}
    want = {rid: _toy2_plain(raw, weights, toks) for rid, toks in reqs.items()}
    for cut in ("fixed", "ragged", "mixed"):
        steps = {"fixed": lambda r: _fixed_portions(r, 8, 30), "ragged": ru.ragged, "mixed": ru.mixed}[cut](reqs)
        pages = ru.max_live_tokens(steps, 64) // 8
        n_groups = len({m for m in mixers if m in ("attention", "window", "latent")})
        # pools of different sizes: the windowed group needs far fewer pages than the others
        counts = [pages if m != "window" else max(16, pages // 2) for m in mixers if m in ("attention", "window", "latent")]
        runner = ModelRunner(cfg, weights, dtype=dtype, page_size=8, num_pages=counts, max_requests=4)
        assert [p.num_pages for p in runner.cache.pools] == counts and len(counts) == n_groups
        assert (runner.decode_graphs_ok, runner.portion_graphs_ok) == (decode_graphs, portion_graphs)
        runner.portion_graph_after = 2
        got = ru.run_trace(runner, steps)
        assert len(got) == sum(len(t) for t in reqs.values())
        ru.compare(got, want, dtype, label=f"toy2/{'+'.join(mixers)}/{cut}/{dtype}")
        if cut == "fixed":
            assert bool(runner._graphs) == decode_graphs, "single-token steps: captured exactly when every part allows it"
            assert bool(runner._portion_graphs) == (portion_graphs and dtype == "bfloat16")
        runner.cache.check_consistency()
        assert all(p.num_free == p.num_pages for p in runner.cache.pools)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_another_embedding_and_another_head(tmp_path, dtype):
    """The two ends of the model are registered parts as well: an embedding that scales its rows
    and a head that caps its logits, defined here, in a model whose steps are captured too."""
    from nanoinfer_b200.config import load_config
    from nanoinfer_b200.engine import ModelRunner
    from nanoinfer_b200.weights import load_weights, write_random_model
    _register_more_toys()
    raw = dict(_toy2_raw(("attention", "window")), embed_scale=3.0, soft_cap=2.0)
    d = str(tmp_path / "toy2e")
    write_random_model(d, raw, seed=8, std=0.08)
    cfg = load_config(d)
    weights = load_weights(d, cfg)
    reqs = {f"e{i}": random_tokens(raw["vocab"], n, 500 + i) for i, n in enumerate([40, 75, 21])}
    want = {rid: _toy2_plain(raw, weights, toks) for rid, toks in reqs.items()}
    assert max(w.abs().max().item() for w in want.values()) > 0.8 * raw["soft_cap"], "the cap must bite"
    for cut in (ru.tail_by_token, ru.mixed):
        steps = cut(reqs)
        runner = ModelRunner(cfg, weights, dtype=dtype, page_size=8, num_pages=ru.max_live_tokens(steps, 64) // 8,
                             max_requests=4)
        assert type(runner.model.embedding).__name__ == "ScaledTable" and type(runner.model.head).__name__ == "SoftCapHead"
        assert runner.decode_graphs_ok
        ru.compare(ru.run_trace(runner, steps), want, dtype, label=f"toy ends/{cut.__name__}/{dtype}")
        assert runner._graphs


def test_a_windowed_group_gets_a_pool_of_its_own_size(tmp_path):
    """One page count for the runner: the group that keeps all keys gets it, a windowed group no
    more than its requests can hold (window + the largest portion, per request)."""
    from nanoinfer_b200.config import load_config
    from nanoinfer_b200.engine import ModelRunner
    from nanoinfer_b200.weights import load_weights, write_random_model
    _register_more_toys()
    raw = _toy2_raw(("attention", "window"))
    d = str(tmp_path / "toy2w")
    write_random_model(d, raw, seed=7, std=0.08)
    cfg = load_config(d)
    weights = load_weights(d, cfg)
    runner = ModelRunner(cfg, weights, dtype="float32", page_size=8, num_pages=400, max_requests=4, max_portion_tokens=24)
    full, windowed = runner.cache.pools
    assert full.num_pages == 400 and windowed.num_pages == 4 * (-(-(20 + 24) // 8) + 2)
    assert runner.caches[0].k_pages.shape[0] == 400 and runner.caches[1].k_pages.shape[0] == windowed.num_pages
    reqs = {f"w{i}": random_tokens(raw["vocab"], n, 400 + i) for i, n in enumerate([300, 180, 250, 90])}
    steps = ru.mixed(reqs, prefill_sizes=(24, 5, 13, 24, 2))
    got = ru.run_trace(runner, steps)
    ru.compare(got, {rid: _toy2_plain(raw, weights, toks) for rid, toks in reqs.items()}, "float32", label="window pool")
    runner.cache.check_consistency()
