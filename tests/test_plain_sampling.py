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
