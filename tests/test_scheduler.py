"""The scheduler's decisions and the engine loop, on the host with a fake runner."""
import pytest

from fakes import ArgmaxSampler, FakeFeedingRunner, FakeRunner, expected_continuation
from nanoinfer_b200.engine import Engine, EngineConfig, RequestState
from nanoinfer_b200.sampling import SamplingParams


def make(runner=None, **cfg):
    runner = runner or FakeRunner()
    return Engine(runner, ArgmaxSampler(), EngineConfig(**cfg)), runner


def test_fcfs_chunks_under_token_budget():
    eng, runner = make(FakeRunner(num_pages=64, max_tokens=128), prefill_chunk_size=8, max_num_batched_tokens=12)
    a = eng.add_request(list(range(1, 21)), 3)      # 20 tokens
    b = eng.add_request(list(range(1, 6)), 3)       # 5 tokens
    eng.step()
    assert runner.steps[-1] == [(a, 8, 0), (b, 4, 0)]            # a's chunk, b gets what is left of 12
    eng.step()
    assert runner.steps[-1] == [(a, 8, 8), (b, 1, 4)]            # b's last prompt token: it emits
    assert len(eng.get_request_result(b)) == 1 and eng.get_request_result(a) == []
    eng.step()
    assert runner.steps[-1] == [(a, 4, 16), (b, 1, 5)]           # a finishes its prompt, b decodes
    assert len(eng.get_request_result(a)) == 1 and len(eng.get_request_result(b)) == 2
    eng.run()
    for rid, prompt in ((a, list(range(1, 21))), (b, list(range(1, 6)))):
        assert eng.get_request_result(rid) == expected_continuation(prompt, 3, 50)
        assert eng.get_request(rid).state == RequestState.FINISHED
        assert eng.get_request(rid).finish_reason == "length"
    runner.cache.check_consistency()
    assert runner.cache.num_free_pages() == 64 and runner.cache.num_free_slots == 4


def test_decoding_requests_keep_their_token_when_the_budget_is_tight():
    eng, runner = make(FakeRunner(num_pages=64, max_tokens=128), prefill_chunk_size=16, max_num_batched_tokens=6)
    a = eng.add_request([1, 2, 3], 8)
    eng.step()                                       # a: whole prompt, emits
    b = eng.add_request(list(range(1, 30)), 2)
    eng.step()
    assert runner.steps[-1] == [(a, 1, 3), (b, 5, 0)]            # 1 set aside for a, 5 left for b
    eng.run()
    assert eng.get_request_result(a) == expected_continuation([1, 2, 3], 8, 50)


def test_batch_size_and_sequence_limits():
    eng, runner = make(FakeRunner(num_pages=64, max_requests=4, max_tokens=64), max_batch_size=2, max_sequences=3)
    ids = [eng.add_request([i + 1, i + 2], 4) for i in range(5)]
    eng.step()
    assert [r for r, _, _ in runner.steps[-1]] == ids[:2]        # max_batch_size
    st = eng.get_scheduler_stats()
    assert (st.num_running, st.num_waiting, st.total_requests) == (2, 3, 5)
    eng.run()
    for i, rid in enumerate(ids):
        assert eng.get_request_result(rid) == expected_continuation([i + 1, i + 2], 4, 50)
    assert eng.get_scheduler_stats().num_finished == 5
    assert max(len(s) for s in runner.steps) <= 2


def test_stop_token_finishes_and_frees():
    prompt = [3, 4]
    first = expected_continuation(prompt, 1, 50)[0]
    runner = FakeRunner()
    eng = Engine(runner, ArgmaxSampler(), EngineConfig(), stop_token_ids=[first])
    rid = eng.add_request(prompt, 10)
    eng.run()
    assert eng.get_request_result(rid) == [first] and eng.get_request(rid).finish_reason == "stop"
    assert runner.cache.num_free_pages() == 16


def test_out_of_pages_preempts_the_latest_and_recomputes():
    # 6 pages of 4 tokens: two requests of 8 prompt tokens fill 4 pages, then both grow
    eng, runner = make(FakeRunner(num_pages=6, page_size=4, max_tokens=24), prefill_chunk_size=8)
    a = eng.add_request(list(range(1, 9)), 10)
    b = eng.add_request(list(range(2, 10)), 10)
    eng.run()
    ra, rb = eng.get_request(a), eng.get_request(b)
    assert ra.num_preemptions == 0 and rb.num_preemptions >= 1   # the later one gives way
    assert eng.get_request_result(a) == expected_continuation(list(range(1, 9)), 10, 50)
    assert eng.get_request_result(b) == expected_continuation(list(range(2, 10)), 10, 50)
    # after preemption b was recomputed from position 0 with its generated tokens as prompt
    restarts = [s for s in runner.steps for (r, n, start) in s if r == b and start == 0]
    assert len(restarts) >= 2
    assert eng.get_scheduler_stats().num_preemptions == rb.num_preemptions
    runner.cache.check_consistency()
    assert runner.cache.num_free_pages() == 6


def test_a_lone_request_that_outgrows_the_pool_fails_and_the_engine_goes_on():
    eng, runner = make(FakeRunner(num_pages=3, page_size=4, max_tokens=64))
    a = eng.add_request(list(range(1, 9)), 20)       # 8 + 20 tokens > 12 the pool holds
    eng.run()
    ra = eng.get_request(a)
    assert ra.state == RequestState.FAILED and ra.finish_reason == "out_of_pages"
    assert eng.get_request_result(a) == expected_continuation(list(range(1, 9)), 20, 50)[:len(ra.generated_tokens)]
    assert len(ra.generated_tokens) == 5             # positions 8..12: the 13th token found no page
    assert runner.cache.num_free_pages() == 3
    b = eng.add_request([5, 6, 7], 2)                # the engine is still alive
    eng.run()
    assert eng.get_request_result(b) == expected_continuation([5, 6, 7], 2, 50)


def test_requests_that_can_never_run_are_refused_at_once():
    eng, runner = make(FakeRunner(num_pages=4, page_size=4, max_tokens=64))
    with pytest.raises(ValueError, match="does not fit the cache pool"):
        eng.add_request(list(range(1, 20)), 4)
    with pytest.raises(ValueError, match="outside"):
        eng.add_request([1, 99], 4)
    with pytest.raises(ValueError, match="at least one"):
        eng.add_request([], 4)
    eng2, _ = make(FakeRunner(num_pages=64, page_size=4, max_tokens=16))
    with pytest.raises(ValueError, match="no room"):
        eng2.add_request(list(range(1, 17)), 4)
    rid = eng2.add_request(list(range(1, 13)), 100)  # max_new_tokens is cut to what fits
    eng2.run()
    assert len(eng2.get_request_result(rid)) == 4
    assert not eng.has_work()


def test_windowed_group_releases_pages_while_running():
    runner = FakeRunner(num_pages=8, page_size=4, max_tokens=64, window=6)
    eng, _ = make(runner, prefill_chunk_size=4)
    a = eng.add_request(list(range(1, 11)), 20)
    peak = 0
    while eng.has_work():
        eng.step()
        peak = max(peak, runner.cache.pools[1].num_taken)
        runner.cache.check_consistency()
    assert eng.get_request(a).state == RequestState.FINISHED
    assert peak <= 3 and runner.cache.pools[0].num_free == 8


def test_generate_keeps_prompt_order_and_default_params():
    eng, _ = make(FakeRunner(num_pages=64, max_tokens=64))
    prompts = [[1, 2, 3], [9], [4, 4, 4, 4, 4]]
    out = eng.generate(prompts, max_new_tokens=3, sampling_params=SamplingParams.greedy())
    assert out == [expected_continuation(p, 3, 50) for p in prompts]
    assert SamplingParams().temperature == 1.0 and SamplingParams().top_k == -1
    assert SamplingParams().top_p == 1.0 and SamplingParams().seed == -1
    assert SamplingParams.greedy().use_greedy() and not SamplingParams().use_greedy()


# ---- overlapped steps: a decode step is launched before the previous step's tokens are read ----

def test_overlapped_steps_give_the_same_tokens_one_call_later():
    prompts = [[3, 1, 4], [1, 5, 9, 2, 6], [5, 3]]
    runner = FakeFeedingRunner(num_pages=64, max_tokens=128)
    eng, _ = make(runner)
    ids = [eng.add_request(p, 9) for p in prompts]
    first = eng.step()                       # prompts: nothing in flight before, tokens stay in flight
    assert first == [] and eng.has_work()
    second = eng.step()                      # launched from the ids in flight, then those are reported
    assert sorted(o.request_id for o in second) == ids and runner.fed_steps == 1
    eng.run()
    for rid, p in zip(ids, prompts):
        assert eng.get_request_result(rid) == expected_continuation(p, 9, 50)
        assert eng.get_request(rid).finish_reason == "length"
    assert runner.fed_steps >= 6 and not eng.has_work()
    runner.cache.check_consistency()
    assert runner.cache.num_free_pages() == 64 and runner.cache.num_free_slots == 4


def test_overlapped_steps_drop_the_token_run_past_a_stop_token():
    prompt = [2, 7, 1]
    free_run = expected_continuation(prompt, 12, 50)
    stop = free_run[5]
    want = free_run[:free_run.index(stop) + 1]
    runner = FakeFeedingRunner(num_pages=64, max_tokens=128)
    eng, _ = make(runner)
    eng.stop_token_ids = (stop,)
    a = eng.add_request(prompt, 12)
    other = eng.add_request([9, 9, 8], 12)
    eng.run()
    assert eng.get_request_result(a) == want and eng.get_request(a).finish_reason == "stop"
    assert eng.get_request_result(other) == expected_continuation([9, 9, 8], 12, 50, stop=(stop,))
    assert runner.fed_steps > 0
    runner.cache.check_consistency()
    assert runner.cache.num_free_pages() == 64


def test_overlapped_steps_read_first_when_the_batch_changes():
    """A request that arrives, a request that ends by length and a page shortage all make the
    engine read the tokens in flight before it decides."""
    runner = FakeFeedingRunner(num_pages=6, page_size=4, max_tokens=24)
    eng, _ = make(runner, prefill_chunk_size=8)
    a = eng.add_request([1, 2, 3], 14)
    eng.step(); eng.step(); eng.step()
    fed = runner.fed_steps
    assert fed == 2
    b = eng.add_request([4, 5, 6, 7, 8], 14)         # waiting: the next step is not a repeat
    eng.step()
    assert runner.fed_steps == fed and [r for r, _, _ in runner.steps[-1]] == [a, b]
    eng.run()                                         # 6 pages of 4 cannot hold 17 + 19 tokens: preemption
    assert eng.get_scheduler_stats().num_preemptions >= 1
    assert eng.get_request_result(a) == expected_continuation([1, 2, 3], 14, 50)
    assert eng.get_request_result(b) == expected_continuation([4, 5, 6, 7, 8], 14, 50)
    runner.cache.check_consistency()
    assert runner.cache.num_free_pages() == 6


def test_overlap_can_be_switched_off():
    runner = FakeFeedingRunner(num_pages=64, max_tokens=128)
    eng, _ = make(runner, overlap_steps=False)
    a = eng.add_request([1, 2, 3], 5)
    assert [o.request_id for o in eng.step()] == [a]
    eng.run()
    assert runner.fed_steps == 0 and eng.get_request_result(a) == expected_continuation([1, 2, 3], 5, 50)


@pytest.mark.parametrize("overlap", [False, True])
def test_a_device_error_word_fails_the_running_requests_and_the_engine_goes_on(overlap):
    """The runner's error word (set by a kernel that gave up a bounded wait) is read with every
    step's sampled ids: the step raises, the running requests fail and give back what they hold,
    a waiting request is untouched, and after the word is cleared the engine serves on."""
    import torch
    from nanoinfer_b200.kernels.ops import KernelError
    runner = FakeFeedingRunner(num_pages=64, max_tokens=128) if overlap else FakeRunner(num_pages=64, max_tokens=128)
    runner.error_word = torch.zeros(1, dtype=torch.int32)
    eng, _ = make(runner, max_sequences=2, overlap_steps=overlap)
    a = eng.add_request([1, 2, 3], 10)
    b = eng.add_request([4, 5], 10)
    c = eng.add_request([7, 7, 7], 6)                 # waits: only two requests run at once
    for _ in range(3):
        eng.step()
    assert eng.get_request(c).state == RequestState.WAITING
    runner.error_word[0] = 13                          # "a kernel gave up" during the step that comes next
    with pytest.raises(KernelError, match="code 13.*softmax"):
        for _ in range(3):
            eng.step()
    assert int(runner.error_word[0]) == 0              # cleared, so that later steps are judged on their own
    for rid in (a, b):
        assert eng.get_request(rid).state == RequestState.FAILED
        assert eng.get_request(rid).finish_reason == "device_error"
    assert eng.get_request(c).state in (RequestState.WAITING, RequestState.RUNNING)   # admitted after the error at the earliest
    eng.run()                                          # no second report; the waiting request is served
    assert eng.get_request_result(c) == expected_continuation([7, 7, 7], 6, 50)
    d = eng.add_request([1, 2, 3], 4)
    eng.run()
    assert eng.get_request_result(d) == expected_continuation([1, 2, 3], 4, 50)
    runner.cache.check_consistency()
    assert runner.cache.num_free_pages() == 64 and runner.cache.num_free_slots == 4
