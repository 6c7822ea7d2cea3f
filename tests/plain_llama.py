"""A plain, slow Llama for the tests: whole sequences, no cache, FP32 on the CPU, one
function per part.  It shares no code with the package: it reads the config.json
dictionary itself and takes weights as {safetensors name: tensor}.

Written from the reference's formulas; every function cites where the reference computes
the same thing (paths relative to the reference project).  Its agreement with the reference rests
on tests/golden/: whole-model logits of the reference's own Python model (tools/model.py;
test_plain_vs_golden.py), and outputs of the reference's own C++ CPU kernels, compiled unchanged,
for what that model lacks - the llama3 frequency rule and sin/cos table, the rotation of adjacent
pairs, attention over a paged cache and of a portion in mid-sequence (test_reference_kernels.py).

Deliberate difference from the reference: its attention softmax divides by (sum + 1e-6)
(src/op/kernels/cpu/prefill_attention_kernel.cpp:133); this one divides by the sum.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

# The precision the plain implementation computes in.  float32 is what the reference computes in;
# float64 serves as the exact value when the rounding of a 32-bit computation itself is what a test
# measures (at the full model size, where sums of 8,192 terms through 16 layers no longer agree to
# 1e-4 between two correct 32-bit implementations that add in different orders).
DTYPE = torch.float32


class precision:
    """with plain.precision(torch.float64): ... - compute in another precision for a while."""

    def __init__(self, dtype):
        self.dtype = dtype

    def __enter__(self):
        global DTYPE
        self.before, DTYPE = DTYPE, self.dtype

    def __exit__(self, *exc):
        global DTYPE
        DTYPE = self.before
        return False


def embedding(table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """h[t] = E[tok[t]]  (src/op/kernels/cpu/embedding_kernel.cpp:30-50)."""
    return table.to(DTYPE)[tokens.long()]


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * g, eps inside the root
    (src/op/kernels/cuda/rmsnorm_kernel.cu:49-104, line 79; tools/model.py:34-39)."""
    x = x.to(DTYPE)
    inv = torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (x * inv) * gain.to(DTYPE)


def rope_inv_freq(rotary_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """Inverse frequencies with the optional llama3 rule, FP32 throughout
    (src/op/kernels/cpu/rope_kernel.cpp:117-139)."""
    f32 = torch.float32        # frequencies and angles are 32-bit numbers by definition, whatever DTYPE is
    idx = torch.arange(0, rotary_dim, 2, dtype=f32)
    freq = 1.0 / torch.pow(torch.tensor(theta, dtype=f32), idx / rotary_dim)
    if scaling is not None and scaling.get("rope_type", scaling.get("type")) == "llama3":
        factor = torch.tensor(float(scaling["factor"]), dtype=f32)
        low = torch.tensor(float(scaling["low_freq_factor"]), dtype=f32)
        high = torch.tensor(float(scaling["high_freq_factor"]), dtype=f32)
        orig = torch.tensor(float(scaling["original_max_position_embeddings"]), dtype=f32)
        wavelen = torch.tensor(2.0 * math.pi, dtype=f32) / freq
        smooth = (orig / wavelen - low) / (high - low)
        blended = (1.0 - smooth) * freq / factor + smooth * freq
        freq = torch.where(wavelen >= orig / low, freq / factor,
                           torch.where(wavelen > orig / high, blended, freq))
    return freq


def rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, pairing: str) -> torch.Tensor:
    """Rotate x [T, H, hd] at the given positions.  angle = float(pos) * freq in FP32.
    "interleaved": pairs (2i, 2i+1) (src/op/kernels/cpu/rope_kernel.cpp:68-93);
    "half": pairs (i, i + rot/2), the same rotation for projection rows in the
    safetensors order (the exporter's permutation, tools/export_llama3.py:571-583)."""
    x = x.to(DTYPE)
    rot = inv_freq.numel() * 2
    angle = (positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, :]).to(DTYPE)   # [T, rot/2], FP32 product
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    out = x.clone()
    if pairing == "interleaved":
        a, b = x[..., 0:rot:2], x[..., 1:rot:2]
        out[..., 0:rot:2] = a * cos - b * sin
        out[..., 1:rot:2] = a * sin + b * cos
    elif pairing == "half":
        a, b = x[..., :rot // 2], x[..., rot // 2:rot]
        out[..., :rot // 2] = a * cos - b * sin
        out[..., rot // 2:rot] = a * sin + b * cos
    else:
        raise ValueError(pairing)
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
              window: Optional[int] = None) -> torch.Tensor:
    """Causal grouped-query attention of one whole sequence.  q [T, Hq, hd], k/v [T, Hkv, hd].
    score = (q.k) * scale; query i sees keys j <= i (and j > i - window); softmax with the
    maximum subtracted; out = P V; kv head = q head // (Hq // Hkv)
    (src/op/kernels/cpu/prefill_attention_kernel.cpp:47-159,
    src/op/kernels/cpu/paged_attention_kernel.cpp:44-135)."""
    T, hq, hd = q.shape
    hkv = k.shape[1]
    rep = hq // hkv
    q, k, v = q.to(DTYPE), k.to(DTYPE), v.to(DTYPE)
    out = torch.empty_like(q)
    i = torch.arange(T)
    mask = i[None, :] <= i[:, None]
    if window is not None:
        mask &= i[None, :] > i[:, None] - window
    for h in range(hq):
        kh, vh = k[:, h // rep, :], v[:, h // rep, :]
        s = (q[:, h, :] @ kh.t()) * scale
        s = s.masked_fill(~mask, float("-inf"))
        s = s - s.max(dim=-1, keepdim=True).values
        e = torch.exp(s)
        p = e / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ vh
    return out


def swiglu_ffn(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)), silu(g) = g / (1 + exp(-g))
    (src/model/llama.cpp:364-379, src/op/kernels/cpu/swiglu_kernel.cpp:25-40)."""
    x = x.to(DTYPE)
    g = x @ w_gate.to(DTYPE).t()
    u = x @ w_up.to(DTYPE).t()
    return ((g / (1.0 + torch.exp(-g))) * u) @ w_down.to(DTYPE).t()


def attention_block(x, w, prefix, n_heads, n_kv, hd, positions, inv_freq, pairing, scale, window=None):
    """QKV projections, RoPE on q and k, attention, output projection
    (src/model/llama.cpp:327-356)."""
    T = x.shape[0]
    q = (x @ w[f"{prefix}.q_proj.weight"].to(DTYPE).t()).view(T, n_heads, hd)
    k = (x @ w[f"{prefix}.k_proj.weight"].to(DTYPE).t()).view(T, n_kv, hd)
    v = (x @ w[f"{prefix}.v_proj.weight"].to(DTYPE).t()).view(T, n_kv, hd)
    q = rope(q, positions, inv_freq, pairing)
    k = rope(k, positions, inv_freq, pairing)
    o = attention(q, k, v, scale, window).reshape(T, n_heads * hd)
    return o @ w[f"{prefix}.o_proj.weight"].to(DTYPE).t()


def forward(raw: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    """Logits [T, V] of one whole sequence at positions 0..T-1
    (layer loop of src/model/llama.cpp:245-389)."""
    d = raw["hidden_size"]
    n_heads = raw["num_attention_heads"]
    n_kv = raw.get("num_key_value_heads") or n_heads
    hd = raw.get("head_dim") or d // n_heads
    eps = raw.get("rms_norm_eps", 1e-5)
    pairing = raw.get("rope_pairing", "half")
    inv_freq = rope_inv_freq(hd, raw.get("rope_theta", 10000.0), raw.get("rope_scaling"))
    scale = 1.0 / math.sqrt(hd)
    tok = torch.as_tensor(list(tokens), dtype=torch.long)
    positions = torch.arange(tok.numel())
    h = embedding(w["model.embed_tokens.weight"], tok)
    for i in range(raw["num_hidden_layers"]):
        p = f"model.layers.{i}"
        x = rms_norm(h, w[f"{p}.input_layernorm.weight"], eps)
        h = h + attention_block(x, w, f"{p}.self_attn", n_heads, n_kv, hd, positions, inv_freq,
                                pairing, scale)
        x = rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps)
        h = h + swiglu_ffn(x, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                           w[f"{p}.mlp.down_proj.weight"])
    h = rms_norm(h, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if raw.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return h @ head.to(DTYPE).t()


def greedy_generate(raw: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], n_new: int) -> List[int]:
    """Arg-max continuation, ties to the lowest id (src/op/kernels/cpu/argmax_kernel.cpp:20-40).
    Recomputes the whole sequence for every token."""
    seq = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward(raw, w, seq)[-1]
        t = int(torch.argmax(logits))  # torch returns the first maximal index
        out.append(t)
        seq.append(t)
    return out


def permute_half_to_interleaved(wt: torch.Tensor, n_heads: int) -> torch.Tensor:
    """Reorder the rows of a q/k projection stored in the safetensors ("half") order into
    the interleaved order (what tools/export_llama3.py:571-573 does on export)."""
    out_dim, in_dim = wt.shape
    hd = out_dim // n_heads
    return wt.view(n_heads, 2, hd // 2, in_dim).transpose(1, 2).reshape(out_dim, in_dim)
