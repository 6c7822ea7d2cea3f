"""The plain implementation against the reference project's own C++ CPU kernels, for the formulas
that its Python model does not contain: the llama3 frequency rule and the sin/cos table, the
rotation of adjacent pairs, attention of single tokens over a paged cache and attention of a
prompt portion that starts in mid-sequence.

The kernels' outputs are stored in tests/golden/reference_cpu_kernels.npz (made by
tests/golden/make_kernel_golden.py from the unchanged sources).  With NANOINFER_REFERENCE set to
the reference project's path the kernels are compiled and run again and must reproduce the file.
"""
import math
import os
import tempfile

import numpy as np
import pytest
import torch

import plain_llama as plain
from golden import make_kernel_golden as mk

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_cpu_kernels.npz")


@pytest.fixture(scope="module")
def gold():
    return dict(np.load(GOLDEN))


def _scaling(sc):
    if sc is None:
        return None
    return {"rope_type": "llama3", "factor": sc[0], "low_freq_factor": sc[1], "high_freq_factor": sc[2],
            "original_max_position_embeddings": sc[3]}


@pytest.mark.parametrize("name,hd,theta,sc,n_pos", mk.ROPE_CASES)
def test_rope_frequencies_and_table(gold, name, hd, theta, sc, n_pos):
    """sin_cos_cache_calc_cpu (src/op/kernels/cpu/rope_kernel.cpp:106-153): value of pair i at
    columns 2i and 2i + 1, angle = float(pos) * freq."""
    inv_freq = plain.rope_inv_freq(hd, theta, _scaling(sc))
    if sc is not None:
        # all three branches of the rule occur among this case's frequencies
        wavelen = 2.0 * math.pi / (1.0 / np.power(np.float32(theta), np.arange(0, hd, 2, dtype=np.float32) / hd))
        low_wl, high_wl = sc[3] / sc[1], sc[3] / sc[2]
        assert (wavelen >= low_wl).any() and (wavelen <= high_wl).any() and ((wavelen < low_wl) & (wavelen > high_wl)).any()
    rows = torch.from_numpy(gold[f"rope/{name}/sin_rows"]).float()
    angle = rows[:, None] * inv_freq[None, :]
    for fn, key in ((torch.sin, "sin"), (torch.cos, "cos")):
        table = torch.from_numpy(gold[f"rope/{name}/{key}"])
        assert torch.equal(table[:, 0::2], table[:, 1::2])
        # a frequency that is one unit in the last place off moves the angle by pos * freq * 2^-23
        tol = 1e-6 + angle.abs() * 2.4e-7
        err = (fn(angle) - table[:, 0::2]).abs()
        assert bool((err <= tol).all()), f"{name}/{key}: largest excess {(err - tol).max().item():.3g}"
    # position 1 holds sin(freq): the frequencies themselves, to FP32 rounding
    one = list(gold[f"rope/{name}/sin_rows"]).index(1)
    torch.testing.assert_close(torch.sin(inv_freq), torch.from_numpy(gold[f"rope/{name}/sin"])[one, 0::2], rtol=3e-7, atol=1e-9)


@pytest.mark.parametrize("name,hd,theta,sc,n_pos", mk.ROPE_CASES)
def test_rotation_of_adjacent_pairs(gold, name, hd, theta, sc, n_pos):
    """rope_kernel_cpu (src/op/kernels/cpu/rope_kernel.cpp:39-96)."""
    inv_freq = plain.rope_inv_freq(hd, theta, _scaling(sc))
    pos = torch.from_numpy(gold[f"rope/{name}/pos"]).long()
    for which in ("q", "k"):
        x = torch.from_numpy(gold[f"rope/{name}/{which}_in"])
        n = x.shape[0]
        got = plain.rope(x.view(n, -1, hd), pos, inv_freq, "interleaved").reshape(n, -1)
        torch.testing.assert_close(got, torch.from_numpy(gold[f"rope/{name}/{which}_out"]), rtol=1e-5, atol=1e-4)


def _sequence_from_cache(cache, table_row, length, block):
    """[length, kv heads, head size] from a cache laid out [block, slot, kv head, head size]."""
    return torch.stack([torch.from_numpy(cache[table_row[t // block], t % block]) for t in range(length)])


@pytest.mark.parametrize("name,hq,hkv,hd,bs,lens", mk.DECODE_CASES)
def test_attention_of_single_tokens_over_pages(gold, name, hq, hkv, hd, bs, lens):
    """paged_attention_kernel_cpu (src/op/kernels/cpu/paged_attention_kernel.cpp:44-135); it divides
    by (sum + 1e-6), the plain implementation by the sum: a relative difference of at most 1e-6."""
    q = torch.from_numpy(gold[f"decode/{name}/q"])
    for b, length in enumerate(lens):
        k = _sequence_from_cache(gold[f"decode/{name}/k_cache"], gold[f"decode/{name}/table"][b], length, bs)
        v = _sequence_from_cache(gold[f"decode/{name}/v_cache"], gold[f"decode/{name}/table"][b], length, bs)
        q_full = torch.zeros(length, hq, hd)
        q_full[-1] = q[b].view(hq, hd)
        got = plain.attention(q_full, k, v, 1.0 / math.sqrt(hd))[-1].reshape(-1)
        torch.testing.assert_close(got, torch.from_numpy(gold[f"decode/{name}/out"])[b], rtol=1e-5, atol=3e-6)


@pytest.mark.parametrize("name,hq,hkv,hd,bs,start,chunk", mk.PREFILL_CASES)
def test_attention_of_a_prompt_portion(gold, name, hq, hkv, hd, bs, start, chunk):
    """prefill_attention_kernel_cpu (src/op/kernels/cpu/prefill_attention_kernel.cpp:47-159): writes
    the portion's keys and values into its pages, then query i sees keys 0 .. start + i."""
    ctx = start + chunk
    k = torch.from_numpy(gold[f"prefill/{name}/k_all"]).view(ctx, hkv, hd)
    v = torch.from_numpy(gold[f"prefill/{name}/v_all"]).view(ctx, hkv, hd)
    q_full = torch.zeros(ctx, hq, hd)
    q_full[start:] = torch.from_numpy(gold[f"prefill/{name}/q"]).view(chunk, hq, hd)
    got = plain.attention(q_full, k, v, 1.0 / math.sqrt(hd))[start:].reshape(chunk, -1)
    torch.testing.assert_close(got, torch.from_numpy(gold[f"prefill/{name}/out"]), rtol=1e-5, atol=3e-6)
    # the page write: token t lies in page table[t // block], slot t % block
    after = _sequence_from_cache(gold[f"prefill/{name}/k_cache_after"], gold[f"prefill/{name}/table"][0], ctx, bs)
    assert torch.equal(after, k)


@pytest.mark.skipif(not os.environ.get("NANOINFER_REFERENCE"), reason="NANOINFER_REFERENCE (path of the reference project) is not set")
def test_the_stored_outputs_are_what_the_reference_kernels_compute():
    with tempfile.TemporaryDirectory() as work:
        data = mk.generate(mk.build(os.environ["NANOINFER_REFERENCE"], work))
    stored = dict(np.load(GOLDEN))
    for key, val in data.items():
        if key.endswith("/sin") or key.endswith("/cos"):
            val = val[stored[key + "_rows"]]
        np.testing.assert_allclose(val, stored[key], rtol=1e-6, atol=1e-7, err_msg=key)
