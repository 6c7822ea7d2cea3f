"""A bounded wait that runs out: the kernel records where it gave up and RETURNS, the host sees
the record, and the next launch is an ordinary one.

The waits of the tcgen05 kernels (on mbarriers, between the loader, the MMA issuer and the
epilogue or softmax warps) are bounded in clock ticks.  For these tests the limit is set to about
a millisecond and the kernels are told to wait once more at their end, for a phase that nothing
completes: the wait runs out by itself.  Nothing traps, faults or spins without a bound.
"""
import math

import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SHORT_LIMIT = 2_000_000      # clock ticks: about a millisecond


def _randn(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).to(DEV)


def _product(ops, module):
    """The smallest product the module takes; returns (result, plain result)."""
    m = {"gemm_tc": 128, "gemm_tc2": 256, "gemm_swap_tc": 16}[module]
    n, k = 256, 128
    a, b = _randn(m, k, seed=1), _randn(n, k, seed=2, scale=0.1)
    out = torch.zeros(m, n, dtype=torch.float32, device=DEV)
    if module == "gemm_swap_tc":
        need = ops.gemm_swap_scratch(m, n, k)
        scratch = torch.zeros(max(need, 1), dtype=torch.float32, device=DEV)
        tickets = torch.zeros(-(-n // 128), dtype=torch.int32, device=DEV)
        ops.gemm_swap_tc(a, b, out, ops.STORE_F32, scratch, tickets)
    else:
        ops.gemm_tc(a, b, out, ops.STORE_F32, kernel="pair" if module == "gemm_tc2" else "single")
    return out, a.float() @ b.float().t()


def _attention(ops):
    n_q, n_kv, hd, page, n = 2, 1, 64, 16, 40
    q = _randn(n, n_q * hd, seed=3)
    k, v = _randn(n, n_kv, hd, seed=4), _randn(n, n_kv, hd, seed=5)
    pages = -(-n // page)
    k_pages = torch.zeros(pages, n_kv, page, hd, dtype=torch.bfloat16, device=DEV)
    v_pages = torch.zeros_like(k_pages)
    for t in range(n):
        k_pages[t // page, :, t % page] = k[t]
        v_pages[t // page, :, t % page] = v[t]
    i32 = dict(dtype=torch.int32, device=DEV)
    out = torch.zeros_like(q)
    ops.attention_prefill(q, k_pages, v_pages, out, torch.zeros(1, **i32), torch.zeros(1, **i32), 1,
                          torch.tensor([0, n], **i32), torch.tensor([n], **i32),
                          torch.arange(pages, **i32).view(1, pages), n_q, n_kv, hd, page, None, 1.0 / math.sqrt(hd),
                          kernel="tc")
    want = plain.attention(q.cpu().view(n, n_q, hd), k.cpu(), v.cpu(), 1.0 / math.sqrt(hd)).reshape(n, n_q * hd)
    return out, want


CODES = {"gemm_tc": 3, "gemm_tc2": 3, "gemm_swap_tc": 23, "attention_prefill_tc": 13}


@pytest.mark.parametrize("module", sorted(CODES))
def test_a_wait_that_runs_out_is_recorded_and_the_kernel_returns(module):
    from nanoinfer_b200.kernels import ops
    run = (lambda: _attention(ops)) if module == "attention_prefill_tc" else (lambda: _product(ops, module))
    run()                                     # loads the library; an ordinary launch leaves no record
    torch.cuda.synchronize()
    ops.check_device_errors()
    ops.set_wait_limit(module, SHORT_LIMIT, extra_wait=True)
    try:
        got, want = run()
        torch.cuda.synchronize()              # returns: the kernel gave up its wait and ended
        with pytest.raises(ops.KernelError, match=f"code {CODES[module]}"):
            ops.check_device_errors()
        # the work itself was done before the extra wait
        torch.testing.assert_close(got.cpu().float(), want.cpu(), rtol=2e-2, atol=2e-2)
    finally:
        ops.set_wait_limit(module, 0, extra_wait=False)
    ops.check_device_errors()                 # the record was cleared by the check above
    got, want = run()                         # tensor memory was given back: the next launch is an ordinary one
    torch.cuda.synchronize()
    ops.check_device_errors()
    torch.testing.assert_close(got.cpu().float(), want.cpu(), rtol=2e-2, atol=2e-2)


def test_the_engine_reports_a_wait_that_ran_out_and_goes_on(model_dirs):
    """Through generation: the prefill attention of a prompt gives up a wait; Engine.step raises a
    KernelError that names the kernel, the request fails, and the next request is served."""
    from nanoinfer_b200 import Engine, SamplingParams
    from nanoinfer_b200.kernels import ops
    from helpers import load_plain, random_tokens
    raw, w = load_plain(model_dirs["d"])
    eng = Engine.from_model_dir(model_dirs["d"], dtype="bfloat16", block_size=16, num_cache_blocks=64, max_sequences=4)
    eng.stop_token_ids = ()
    prompt = random_tokens(raw["vocab_size"], 40, 1)
    first = eng.generate([prompt], max_new_tokens=4, sampling_params=SamplingParams.greedy())[0]
    ops.set_wait_limit("attention_prefill_tc", SHORT_LIMIT, extra_wait=True)
    try:
        rid = eng.add_request(prompt, 4, SamplingParams.greedy())
        with pytest.raises(ops.KernelError, match="code 13"):
            eng.run()
    finally:
        ops.set_wait_limit("attention_prefill_tc", 0, extra_wait=False)
    assert eng.get_request(rid).finish_reason == "device_error"
    assert eng.generate([prompt], max_new_tokens=4, sampling_params=SamplingParams.greedy())[0] == first
    eng.runner.cache.check_consistency()
    assert eng.runner.cache.num_free_pages() == 64
