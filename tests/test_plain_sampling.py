"""The plain selection itself (no GPU)."""
import torch

import plain_sampling as ps


def test_philox_known_answer():
    # Philox4x32-10 with an all-zero counter and key (first word of the published test vector)
    assert ps.philox_first_word(0, 0) == 0x6627E8D5
    assert 0.0 < ps.uniform(3, 5) < 1.0 and ps.uniform(3, 5) != ps.uniform(3, 6) != ps.uniform(4, 5)


def test_filters():
    l = torch.tensor([0.0, 3.0, 1.0, 2.0, -1.0])
    assert ps.sample(l, 0.0)[0] == 1
    assert all(ps.sample(l, 1.0, top_k=1, seed=s)[0] == 1 for s in range(20))
    assert {ps.sample(l, 1.0, top_k=2, seed=s)[0] for s in range(200)} == {1, 3}
    # softmax(l) = [.03, .64, .09, .24, .01]: p = 0.7 keeps {1, 3}; p = 0.5 keeps {1}
    assert {ps.sample(l, 1.0, top_p=0.7, seed=s)[0] for s in range(200)} == {1, 3}
    assert {ps.sample(l, 1.0, top_p=0.5, seed=s)[0] for s in range(50)} == {1}
    # penalty 4 on token 1: 3.0 -> 0.75; on token 4: -1 -> -4
    out = ps.penalise(l, [1, 4, 1], 4.0)
    assert out.tolist() == [0.0, 0.75, 1.0, 2.0, -4.0]
    assert ps.sample(l, 0.0, repetition_penalty=4.0, generated=[1])[0] == 3
    tok, acceptable, cut = ps.sample(l, 1.0, top_p=0.7, seed=1)
    assert acceptable == {tok} and cut > 0.01


def test_sampler_packs_the_rows_parameters_into_one_buffer():
    """The sampler's per-row parameters travel as one buffer of 4-byte words (seeds and token
    counters as 64-bit values first, so that they stay aligned); the views handed to the kernel
    must read back what went in, also when the ring of host buffers comes round."""
    from nanoinfer_b200.sampling import Sampler, SamplingParams
    s = Sampler(vocab_size=100, device=torch.device("cpu"))
    for n in (1, 3, 5, 70):                          # 70 rows outgrow the first buffer
        params = [SamplingParams(temperature=0.5 + r, top_k=r - 1, top_p=1.0 / (r + 1)) for r in range(n)]
        seeds = [(1 << 55) - 1 - r for r in range(n)]
        counts = list(range(10, 10 + n))
        for _ in range(6):                           # more calls than host buffers
            seed_t, count_t, temp_t, top_p_t, top_k_t = s._upload(torch.device("cpu"), params, seeds, counts)
            assert seed_t.dtype == torch.int64 and seed_t.tolist() == seeds
            assert count_t.dtype == torch.int64 and count_t.tolist() == counts
            assert temp_t.dtype == torch.float32 and temp_t.tolist() == [0.5 + r for r in range(n)]
            assert torch.allclose(top_p_t, torch.tensor([1.0 / (r + 1) for r in range(n)]))
            assert top_k_t.dtype == torch.int32 and top_k_t.tolist() == [r - 1 for r in range(n)]
    assert s.h2d_bytes == 6 * 28 * (1 + 3 + 5 + 70)
