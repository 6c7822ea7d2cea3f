"""The entry point that allocates nothing (ni_attention_decode_noalloc), called through its
exported C symbol, against the regular decode attention entry point.

For users of the library who cannot give it scratch memory - a host program that has handed
its whole device budget to its cache pool, a plug-in under a foreign allocator, a decode loop
that must not stall on cudaMalloc - the library keeps the scratch of this one kernel in arrays
of its own image.  This file checks that the variant computes what the regular entry point
computes, on two calls in a row (the second finds the first call's leftovers in the shared
arrays), and that a call beyond the arrays' fixed size is refused instead of run.

It is collected last on purpose, so that a run that stops at the first failure has already
run every other test; it passes alone in a fresh process as well as after the others.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

_I, _F, _P = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
MAX_PARTIAL_FLOATS = 1 << 20        # NI_NOALLOC_MAX_PARTIAL_FLOATS
MAX_TICKETS = 4096                  # NI_NOALLOC_MAX_TICKETS
ERR_STATIC_SCRATCH_TOO_SMALL = -4


def _symbol():
    """The exported C symbol itself, from a handle of its own on the built library (the argument
    types are the ones the package registers for it, checked here against a second declaration)."""
    from nanoinfer_b200.kernels import build, ops
    lib = ctypes.CDLL(build.ensure_built(["attention_decode"])["attention_decode"])
    fn = lib.ni_attention_decode_noalloc
    fn.argtypes = [_P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P]
    fn.restype = _I
    assert ops._SIGNATURES["attention_decode"]["ni_attention_decode_noalloc"] == fn.argtypes
    return fn


def _case(seed, lens, n_q, n_kv, hd, page):
    g = torch.Generator().manual_seed(seed)
    n_seq = len(lens)
    width = max(-(-t // page) for t in lens)
    n_pages = sum(-(-t // page) for t in lens) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((n_seq, width), -1, dtype=torch.int32)
    for s, t in enumerate(lens):
        for i in range(-(-t // page)):
            table[s, i] = perm.pop()
    k_pages = torch.randn(n_pages, n_kv, page, hd, generator=g).to(torch.bfloat16)
    v_pages = torch.randn(n_pages, n_kv, page, hd, generator=g).to(torch.bfloat16)
    q = torch.randn(n_seq, n_q * hd, generator=g).to(torch.bfloat16)
    positions = torch.tensor([t - 1 for t in lens], dtype=torch.int32)
    seq_of = torch.arange(n_seq, dtype=torch.int32)
    return [x.to(DEV) for x in (q, k_pages, v_pages, positions, seq_of, table)]


def test_noalloc_entry_point_matches_the_regular_one_twice_in_a_row():
    from nanoinfer_b200.kernels import ops
    fn = _symbol()
    n_q, n_kv, hd, page = 32, 8, 64, 16
    stream = torch.cuda.current_stream().cuda_stream
    for call, (seed, lens, n_splits) in enumerate([(1, [300, 17, 1024, 64], 5), (2, [90, 513, 33], 3)]):
        q, k_pages, v_pages, positions, seq_of, table = _case(seed, lens, n_q, n_kv, hd, page)
        n = q.shape[0]
        scale = 1.0 / math.sqrt(hd)
        want = torch.zeros_like(q)
        scratch = torch.empty(n * n_q * n_splits * (hd + 2), dtype=torch.float32, device=DEV)
        tickets = torch.zeros(n * n_kv, dtype=torch.int32, device=DEV)
        ops.attention_decode(q, k_pages, v_pages, want, None, n, positions, seq_of, table, n_q, n_kv, hd, page,
                             None, scale, n_splits, scratch, tickets)
        got = torch.zeros_like(q)
        rc = fn(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), got.data_ptr(), None, n,
                positions.data_ptr(), seq_of.data_ptr(), table.data_ptr(), table.shape[1], n_q, n_kv, hd, page,
                0, scale, n_splits, stream)
        assert rc == 0, f"call {call}: ni_attention_decode_noalloc returned {rc}"
        torch.cuda.synchronize()
        # same kernel, same order of sums: the tolerance of the decode attention tests is far
        # more than is needed, the outputs are expected to be identical
        torch.testing.assert_close(got.float(), want.float(), rtol=8e-3, atol=4e-3)
        assert torch.equal(got, want)


def test_noalloc_entry_point_refuses_what_its_arrays_cannot_hold():
    fn = _symbol()
    q, k_pages, v_pages, positions, seq_of, table = _case(3, [40, 50], 32, 8, 64, 16)
    out = torch.full_like(q, 3.0)
    stream = torch.cuda.current_stream().cuda_stream
    # 2 * 32 * n_splits * 66 floats > 2^20 for n_splits = 300
    n_splits = 300
    assert 2 * 32 * n_splits * 66 > MAX_PARTIAL_FLOATS
    rc = fn(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), None, 2, positions.data_ptr(),
            seq_of.data_ptr(), table.data_ptr(), table.shape[1], 32, 8, 64, 16, 0, 0.125, n_splits, stream)
    assert rc == ERR_STATIC_SCRATCH_TOO_SMALL
    torch.cuda.synchronize()
    assert torch.all(out == 3.0)        # nothing was launched


@pytest.mark.parametrize("n_q,n_kv,hd,page,window,listed", [(24, 8, 128, 16, None, False), (32, 8, 64, 16, 200, False),
                                                             (8, 2, 128, 8, 77, True), (32, 8, 64, 16, None, True)])
def test_noalloc_entry_point_with_wide_heads_windows_and_token_lists(n_q, n_kv, hd, page, window, listed):
    """The other kernel variants behind the same entry point: heads of 128, a window of recent keys,
    and a list that picks some of the step's tokens - again two calls in a row."""
    from nanoinfer_b200.kernels import ops
    fn = _symbol()
    stream = torch.cuda.current_stream().cuda_stream
    for seed, lens, n_splits in [(4, [300, 17, 700, 64, 129], 4), (5, [90, 513, 33, 256, 2], 2)]:
        q, k_pages, v_pages, positions, seq_of, table = _case(seed, lens, n_q, n_kv, hd, page)
        picked = torch.tensor([3, 0, 4], dtype=torch.int32, device=DEV) if listed else None
        n = picked.numel() if listed else q.shape[0]
        scale = 1.0 / math.sqrt(hd)
        want = torch.full_like(q, 2.0)
        scratch = torch.empty(n * n_q * n_splits * (hd + 2), dtype=torch.float32, device=DEV)
        tickets = torch.zeros(n * n_kv, dtype=torch.int32, device=DEV)
        ops.attention_decode(q, k_pages, v_pages, want, picked, n, positions, seq_of, table, n_q, n_kv, hd, page,
                             window, scale, n_splits, scratch, tickets)
        got = torch.full_like(q, 2.0)
        rc = fn(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), got.data_ptr(),
                picked.data_ptr() if listed else None, n, positions.data_ptr(), seq_of.data_ptr(), table.data_ptr(),
                table.shape[1], n_q, n_kv, hd, page, window or 0, scale, n_splits, stream)
        assert rc == 0
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float(), want.float(), rtol=8e-3, atol=4e-3)
        assert torch.equal(got, want)
        if listed:
            assert torch.all(got[1] == 2.0) and torch.all(got[2] == 2.0)     # tokens that were not picked stay untouched


def test_noalloc_entry_point_at_and_beyond_its_limits():
    """A call that needs exactly the arrays' size runs; one float more, or one ticket more, is refused."""
    from nanoinfer_b200.kernels import ops
    fn = _symbol()
    stream = torch.cuda.current_stream().cuda_stream
    # 4 tokens x 32 heads x 124 splits x 66 floats = 1,047,552 <= 2^20 < the same with 125 splits
    n_q, n_kv, hd, page = 32, 8, 64, 16
    lens = [8000, 7990, 8100, 64]
    q, k_pages, v_pages, positions, seq_of, table = _case(6, lens, n_q, n_kv, hd, page)
    n = len(lens)
    for n_splits, fits in ((124, True), (125, False)):
        assert (n * n_q * n_splits * (hd + 2) <= MAX_PARTIAL_FLOATS) == fits
        out = torch.full_like(q, 3.0)
        rc = fn(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), None, n, positions.data_ptr(),
                seq_of.data_ptr(), table.data_ptr(), table.shape[1], n_q, n_kv, hd, page, 0, 0.125, n_splits, stream)
        torch.cuda.synchronize()
        if fits:
            assert rc == 0
            want = torch.zeros_like(q)
            scratch = torch.empty(n * n_q * n_splits * (hd + 2), dtype=torch.float32, device=DEV)
            tickets = torch.zeros(n * n_kv, dtype=torch.int32, device=DEV)
            ops.attention_decode(q, k_pages, v_pages, want, None, n, positions, seq_of, table, n_q, n_kv, hd, page,
                                 None, 0.125, n_splits, scratch, tickets)
            torch.cuda.synchronize()
            assert torch.equal(out, want)
        else:
            assert rc == ERR_STATIC_SCRATCH_TOO_SMALL and torch.all(out == 3.0)
    # tickets: 513 tokens x 8 kv heads = 4,104 > 4,096, while the floats fit (513 x 8 heads x 66 x 1 split)
    n_big, few_q = 513, 8
    assert n_big * n_kv > MAX_TICKETS and n_big * few_q * (hd + 2) <= MAX_PARTIAL_FLOATS
    qb = torch.zeros(n_big, few_q * hd, dtype=torch.bfloat16, device=DEV)
    out = torch.full_like(qb, 3.0)
    i32 = dict(dtype=torch.int32, device=DEV)
    rc = fn(qb.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), None, n_big,
            torch.zeros(n_big, **i32).data_ptr(), torch.zeros(n_big, **i32).data_ptr(), table.data_ptr(), table.shape[1],
            few_q, n_kv, hd, page, 0, 0.125, 1, stream)
    torch.cuda.synchronize()
    assert rc == ERR_STATIC_SCRATCH_TOO_SMALL and torch.all(out == 3.0)
