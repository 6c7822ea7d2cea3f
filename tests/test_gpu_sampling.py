"""The sampling kernels against the plain selection, row by row."""
import pytest
import torch

import plain_sampling as ps

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _logits(rows, vocab, seed, scale=3.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(rows, vocab, generator=g) * scale


@pytest.mark.parametrize("vocab", [256, 1000, 128256])
def test_argmax_ties_go_to_the_lowest_id(vocab):
    from nanoinfer_b200.kernels import ops
    l = _logits(5, vocab, 0)
    l[1, 7] = l[1, vocab - 3] = l[1].max() + 1.0     # a tie: the lower id wins
    l[2, :] = 0.5                                    # all equal: id 0
    l[3, vocab - 1] = 100.0                          # the last id
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops.argmax(l.to(DEV), out)
    want = [int(torch.argmax(l[0])), 7, 0, vocab - 1, int(torch.argmax(l[4]))]
    assert out.tolist() == want


CASES = [dict(temperature=1.0), dict(temperature=0.7), dict(temperature=1.5, top_k=5),
         dict(temperature=0.8, top_p=0.9), dict(temperature=1.0, top_k=40, top_p=0.5),
         dict(temperature=0.0), dict(temperature=1.0, top_k=1), dict(temperature=2.0, top_p=0.05),
         dict(temperature=0.9, repetition_penalty=1.3), dict(temperature=0.0, repetition_penalty=2.0)]


@pytest.mark.parametrize("vocab", [4096, 5001, 33007, 128256, 262145])
def test_a_cluster_per_row_selects_the_same_tokens_as_one_block(vocab):
    """Rows of every kind of parameters, at vocabularies that do and do not divide by the cluster's
    eight blocks: the cluster kernel and the one-block kernel agree on every token, bit for bit."""
    from nanoinfer_b200.kernels import ops
    rows = 40
    g = torch.Generator().manual_seed(vocab)
    l = (torch.randn(rows, vocab, generator=g) * 3.0).to(DEV)
    l[3] = 0.25                                                     # all equal: every id as likely
    l[4, :] = -0.0
    l[4, 17] = 0.0                                                  # +0 and -0 tie: the lowest id wins a greedy row
    temps = torch.tensor([[0.0, 0.7, 1.0, 1.5][i % 4] for i in range(rows)], device=DEV)
    temps[4] = 0.0
    ks = torch.tensor([[0, 1, 40, 5000, vocab, 0][i % 6] for i in range(rows)], dtype=torch.int32, device=DEV)
    ps_ = torch.tensor([[1.0, 0.9, 0.5, 0.05, 0.999][i % 5] for i in range(rows)], device=DEV)
    seeds = torch.arange(rows, dtype=torch.int64, device=DEV) * 7919
    counters = torch.arange(rows, dtype=torch.int64, device=DEV) % 5
    outs = []
    for cluster in (True, False):
        ops.sample_by_cluster(cluster)
        out = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
        ops.sample(l, out, temps, ks, ps_, seeds, counters)
        outs.append(out.cpu())
    ops.sample_by_cluster(True)
    assert torch.equal(outs[0], outs[1]), f"rows {torch.nonzero(outs[0] != outs[1]).flatten().tolist()} differ"
    assert int(outs[0].min()) >= 0 and int(outs[0].max()) < vocab and int(outs[0][4]) == 0
    # many draws of one row: different counters give different tokens, the same counter the same token
    many = 64
    rep = l[1:2].expand(many, vocab).contiguous()
    out_a = torch.empty(many, dtype=torch.int32, device=DEV)
    t1 = torch.ones(many, device=DEV)
    z0 = torch.zeros(many, dtype=torch.int32, device=DEV)
    sd = torch.full((many,), 5, dtype=torch.int64, device=DEV)
    ops.sample(rep, out_a, t1, z0, t1, sd, torch.arange(many, dtype=torch.int64, device=DEV))
    assert len(set(out_a.tolist())) > many // 2
    out_b = torch.empty_like(out_a)
    ops.sample(rep, out_b, t1, z0, t1, sd, torch.zeros(many, dtype=torch.int64, device=DEV))
    assert len(set(out_b.tolist())) == 1 and out_b[0] == out_a[0]


@pytest.mark.parametrize("vocab", [384, 1000, 128256])
def test_sampler_matches_plain_selection(vocab):
    from nanoinfer_b200.sampling import Sampler, SamplingParams
    sampler = Sampler(vocab, torch.device(DEV))
    rows = len(CASES) * 3
    l = _logits(rows, vocab, 1)
    params, seeds, idxs, gens = [], [], [], []
    for r in range(rows):
        c = CASES[r % len(CASES)]
        params.append(SamplingParams(**c))
        seeds.append(1000 + r // len(CASES))
        idxs.append(r)
        g = torch.Generator().manual_seed(r)
        gens.append(torch.randint(0, vocab, (20,), generator=g).tolist() + [int(torch.argmax(l[r]))])
    got = sampler.sample(l.clone().to(DEV), params, seeds, idxs, gens).tolist()
    skipped = 0
    for r in range(rows):
        p = params[r]
        tok, acceptable, cut_margin = ps.sample(l[r], p.temperature, p.top_k, p.top_p, p.repetition_penalty,
                                                gens[r], seeds[r], idxs[r])
        if cut_margin < ps.ROUNDING:      # the top-p cut itself is within rounding: two valid kept sets
            skipped += 1
            continue
        assert got[r] in acceptable, f"row {r} {p}: kernel {got[r]}, plain {tok} (acceptable {acceptable})"
    assert skipped <= 1


def test_draws_follow_the_distribution_and_do_not_depend_on_the_batch():
    from nanoinfer_b200.sampling import Sampler, SamplingParams
    vocab, n = 12, 6000
    sampler = Sampler(vocab, torch.device(DEV))
    row = torch.tensor([2.0, 1.0, 0.0, -1.0, 0.5, 1.5, -3.0, 0.0, 0.2, 1.1, -0.5, 0.7])
    l = row.repeat(n, 1)
    sp = SamplingParams(temperature=0.8, seed=5)
    got = sampler.sample(l.to(DEV), [sp] * n, [5] * n, list(range(n))).cpu()
    probs = torch.softmax(row / 0.8, 0)
    freq = torch.bincount(got.long(), minlength=vocab).double() / n
    sigma = torch.sqrt(probs * (1 - probs) / n)
    assert torch.all((freq - probs).abs() <= 5 * sigma + 1e-9)
    # token i of a request is the same alone, in another row, or beside other requests
    alone = sampler.sample(row[None].to(DEV), [sp], [5], [17]).item()
    assert alone == got[17].item()
    mixed = sampler.sample(l[:3].to(DEV), [SamplingParams.greedy(), sp, SamplingParams(seed=9)], [0, 5, 9], [0, 17, 3])
    assert mixed[1].item() == alone and mixed[0].item() == 0
