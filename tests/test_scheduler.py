"""The scheduler's decisions with a scripted executor instead of a model (no GPU)."""

import pytest

from rapid_llm_b200.cache import CacheManager, plan_groups
from rapid_llm_b200.config import EngineConfig
from rapid_llm_b200.engine.scheduler import CacheExhausted, Scheduler
from rapid_llm_b200.parts.base import CacheNeed
from rapid_llm_b200.sampling import SamplingParams


class ScriptedExecutor:
    """Keeps the real cache bookkeeping, returns ``1000 + index of the generated token``."""

    def __init__(self, config: EngineConfig, pages: int, needs=None) -> None:
        groups, _ = plan_groups(needs or [CacheNeed("full", 1, 16)])
        self.cache = CacheManager(groups, page_size=config.page_size, num_pages=pages,
                                  max_num_seqs=config.max_num_seqs, max_seq_len=config.max_seq_len)
        self.steps: list[list[tuple]] = []
        self.stop_after: dict = {}

    def admit(self, request_id):
        return self.cache.admit(request_id) is not None

    def release(self, request_id):
        self.cache.release(request_id)

    def execute(self, entries):
        self.steps.append([(e.request.request_id, e.start, len(e.tokens), e.samples) for e in entries])
        sampled = []
        for entry in entries:
            assert entry.start == self.cache.num_tokens(entry.request.request_id), "a portion must start where the cache ends"
            assert self.cache.reserve(entry.request.request_id, entry.start + len(entry.tokens)), "the plan overbooked the pool"
            assert entry.tokens == entry.request.all_token_ids[entry.start : entry.start + len(entry.tokens)]
            if entry.samples:
                index = len(entry.request.output_token_ids)
                stop = self.stop_after.get(entry.request.request_id)
                sampled.append(7 if stop is not None and index >= stop else 1000 + index)
        for entry in entries:
            self.cache.release_passed(entry.request.request_id)      # as the step function does
        self.cache.check()
        return sampled


def make(pages=64, needs=None, **overrides):
    values = dict(max_seq_len=256, page_size=16, max_num_seqs=4, max_num_batched_tokens=64, max_chunk_size=32)
    values.update(overrides)
    config = EngineConfig(**values)
    executor = ScriptedExecutor(config, pages, needs)
    return Scheduler(executor, config, stop_token_ids=[7]), executor


def greedy(n):
    return SamplingParams.greedy(max_gen_len=n)


def test_prompt_is_cut_into_portions_under_the_chunk_size():
    scheduler, executor = make()
    request = scheduler.add_request(list(range(70)), greedy(3), "a")
    scheduler.run_to_completion()
    assert [step[0][1:] for step in executor.steps] == [(0, 32, False), (32, 32, False), (64, 6, True), (70, 1, True), (71, 1, True)]
    assert request.output_token_ids == [1000, 1001, 1002] and request.finish_reason == "length"
    assert executor.cache.num_free_pages() == 64 and executor.cache.num_free_slots == 4


def test_token_budget_decodes_first_then_resumed_then_new():
    scheduler, executor = make(max_num_batched_tokens=40)
    scheduler.add_request(list(range(10)), greedy(8), "a")
    scheduler.step()                                   # a: whole prompt, samples
    scheduler.add_request(list(range(50)), greedy(2), "b")
    scheduler.add_request(list(range(30)), greedy(2), "c")
    scheduler.step()
    assert executor.steps[-1] == [("a", 10, 1, True), ("b", 0, 32, False), ("c", 0, 7, False)]   # 1 + 32 + 7 = 40
    scheduler.step()
    assert executor.steps[-1] == [("a", 11, 1, True), ("b", 32, 18, True), ("c", 7, 21, False)]
    assert sum(n for _, _, n, _ in executor.steps[-1]) == 40


def test_first_token_comes_from_the_last_portion_and_eos_is_not_appended():
    scheduler, executor = make()
    executor.stop_after["a"] = 2
    request = scheduler.add_request(list(range(5)), greedy(10), "a")
    scheduler.run_to_completion()
    assert request.output_token_ids == [1000, 1001] and request.finish_reason == "eos"
    assert request.first_token_time is not None


def test_admission_is_fcfs_and_bounded_by_slots():
    scheduler, executor = make(max_num_seqs=2, max_num_batched_tokens=256)
    requests = [scheduler.add_request(list(range(4)), greedy(2), name) for name in "abc"]
    scheduler.step()
    assert [e[0] for e in executor.steps[-1]] == ["a", "b"]
    scheduler.step()
    assert [e[0] for e in executor.steps[-1]] == ["a", "b"]      # both finish here
    scheduler.step()
    assert [e[0] for e in executor.steps[-1]] == ["c"]
    scheduler.run_to_completion()
    assert all(r.finish_reason == "length" for r in requests)


def test_waiting_request_waits_for_pages():
    scheduler, executor = make(pages=4, max_num_batched_tokens=256, max_chunk_size=256)
    first = scheduler.add_request(list(range(40)), greedy(3), "a")      # 3 pages
    second = scheduler.add_request(list(range(30)), greedy(3), "b")     # 2 pages: must wait
    scheduler.step()
    assert [e[0] for e in executor.steps[-1]] == ["a"] and second.status == "waiting"
    scheduler.run_to_completion()
    assert first.finish_reason == second.finish_reason == "length"
    assert scheduler.num_preemptions == 0


def test_growth_evicts_the_youngest_which_recomputes_with_its_tokens_folded_in():
    scheduler, executor = make(pages=4, max_num_batched_tokens=256, max_chunk_size=256)
    old = scheduler.add_request(list(range(30)), greedy(20), "old")      # 49 tokens = 4 pages alone
    young = scheduler.add_request(list(range(20)), greedy(30), "young")  # 49 tokens = 4 pages alone
    scheduler.step()                                                      # both prefill: 2 + 2 pages
    assert executor.cache.num_free_pages() == 0
    for _ in range(3):
        scheduler.step()                                                  # old reaches 33 tokens: needs a third page
    assert scheduler.num_preemptions >= 1 and young.num_preemptions >= 1 and old.num_preemptions == 0
    kept = list(young.output_token_ids)
    assert kept, "the evicted request keeps what it generated"
    scheduler.run_to_completion()
    assert old.finish_reason == young.finish_reason == "length"
    assert len(old.output_token_ids) == 20 and len(young.output_token_ids) == 30
    assert young.output_token_ids[: len(kept)] == kept
    assert young.output_token_ids == [1000 + i for i in range(30)]
    recompute = [e for step in executor.steps for e in step if e[0] == "young" and e[1] == 0]
    assert len(recompute) >= 2 and recompute[-1][2] > 20, "the recomputed prompt holds the generated tokens"
    assert executor.cache.num_free_pages() == 4


def test_without_eviction_a_stuck_pool_is_an_error_not_a_spin():
    scheduler, executor = make(pages=4, max_num_batched_tokens=256, max_chunk_size=256, enable_preemption=False)
    scheduler.add_request(list(range(30)), greedy(20), "a")
    scheduler.add_request(list(range(30)), greedy(20), "b")
    with pytest.raises(CacheExhausted):
        scheduler.run_to_completion()


def test_submission_checks():
    scheduler, _ = make(pages=4)
    with pytest.raises(ValueError, match="empty"):
        scheduler.add_request([], greedy(1))
    with pytest.raises(ValueError, match="max_seq_len"):
        scheduler.add_request(list(range(256)), greedy(1))
    with pytest.raises(ValueError, match="pages"):
        scheduler.add_request(list(range(100)), greedy(1))           # 7 pages > 4
    roomy, _ = make(pages=64)
    request = roomy.add_request(list(range(10)), SamplingParams(temperature=0.0, max_gen_len=None))
    assert request.max_new_tokens == 246                                 # None fills the context


def test_whole_prompts_only_when_chunking_is_off():
    scheduler, executor = make(enable_chunked_prefill=False, max_seq_len=64, max_num_batched_tokens=64)
    scheduler.add_request(list(range(50)), greedy(1), "a")
    scheduler.add_request(list(range(40)), greedy(1), "b")
    scheduler.step()
    assert executor.steps[-1] == [("a", 0, 50, True)]                 # b does not fit the budget whole
    scheduler.step()
    assert executor.steps[-1] == [("b", 0, 40, True)]


def test_limits_that_would_leave_a_prompt_waiting_for_ever_are_refused():
    """With chunking off a step must hold the longest prompt; a chunk size of 0 is the older
    switch for the same (``rapid_llm/engine/batch_planner.py:212-233``)."""
    with pytest.raises(ValueError, match="chunked prefill off"):
        EngineConfig(max_seq_len=256, max_num_batched_tokens=64, enable_chunked_prefill=False)
    with pytest.raises(ValueError, match="chunked prefill off"):
        EngineConfig(max_seq_len=256, max_num_batched_tokens=64, max_chunk_size=0)
    folded = EngineConfig(max_seq_len=256, max_num_batched_tokens=256, max_chunk_size=0)
    assert folded.enable_chunked_prefill is False
    with pytest.raises(ValueError, match="max_seq_len"):
        EngineConfig(max_seq_len=1)
    with pytest.raises(ValueError, match="max_chunk_size"):
        EngineConfig(max_chunk_size=-1)


def test_a_refused_prompt_leaves_nothing_of_its_call_in_the_queue():
    """``LLM.generate`` submits its prompts one by one; when one is refused, those before it must not
    stay queued for the next call to run."""
    from rapid_llm_b200.engine.llm import LLM

    scheduler, executor = make()
    llm = object.__new__(LLM)                          # the submission path alone: no device, no model
    llm.scheduler, llm.tokenizer = scheduler, None
    with pytest.raises(ValueError, match="empty"):
        llm._submit([list(range(5)), list(range(9)), []], greedy(2))
    assert not scheduler.has_unfinished() and not scheduler.waiting
    _, requests = llm._submit([list(range(5))], greedy(2))
    scheduler.run_to_completion()
    assert requests[0].output_token_ids == [1000, 1001] and len(executor.steps) == 2


def test_the_references_calling_forms_are_taken():
    """Text first and ids by keyword, ``sampling_params``, ``has_unfinished_requests``, abort by id
    (``rapid_llm/engine/scheduler.py:635-643``)."""
    scheduler, executor = make()
    a = scheduler.add_request("ignored text", sampling_params=greedy(2), request_id="a", prompt_token_ids=list(range(5)))
    b = scheduler.add_request(list(range(9)), greedy(50), "b")
    assert a.prompt_token_ids == list(range(5)) and a.params.max_gen_len == 2
    with pytest.raises(ValueError):
        scheduler.add_request("text alone")
    assert scheduler.has_unfinished_requests()
    scheduler.step()
    scheduler.abort("b")
    scheduler.abort("nobody")                           # unknown ids are not an error
    scheduler.run_to_completion()
    assert not scheduler.has_unfinished_requests()
    assert a.output_token_ids == [1000, 1001] and b.finish_reason == "abort"
    assert executor.cache.num_free_slots == 4


def test_sampling_params_are_validated():
    for bad in (dict(temperature=-1), dict(top_p=0), dict(top_p=1.5), dict(max_gen_len=0), dict(repetition_penalty=0)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)
    assert SamplingParams().temperature == 0.6 and SamplingParams().top_p == 0.9 and SamplingParams().repetition_penalty == 1.1
    assert SamplingParams(stop_on_repeat=False, logprobs=None).stop_on_repeat is False      # the reference's fields are accepted
    with pytest.raises(ValueError):
        SamplingParams(logprobs=5)
    assert SamplingParams(temperature=0).is_greedy


# ------------------------------------------------------------------ running ahead
class RunAheadExecutor(ScriptedExecutor):
    """Adds ``launch``/``collect``: a launched step's tokens are computed when it is collected,
    as on the device, where a token id ``-(row + 1)`` reads row ``row`` of the previous result."""

    def __init__(self, config, pages):
        super().__init__(config, pages)
        self.previous_result: list[int] = []
        self.fed: list[list[int]] = []          # per step, the token ids the model actually saw
        self.collected = 0
        self.launched = 0

    def launch(self, entries):
        self.launched += 1
        self.steps.append([(e.request.request_id, e.start, len(e.tokens), e.samples) for e in entries])
        sampled, fed = [], []
        for entry in entries:
            assert entry.start == self.cache.num_tokens(entry.request.request_id)
            assert self.cache.reserve(entry.request.request_id, entry.start + len(entry.tokens))
            for token in entry.tokens:
                fed.append(self.previous_result[-token - 1] if token < 0 else token)
            if entry.samples:
                index = sum(1 for t in entry.request.output_token_ids)          # stand-ins count
                stop = self.stop_after.get(entry.request.request_id)
                sampled.append(7 if stop is not None and index >= stop else 1000 + index)
        for entry in entries:
            self.cache.release_passed(entry.request.request_id)      # as the step function does
        self.cache.check()
        self.fed.append(fed)
        self.previous_result = sampled
        return (self.launched, sampled)

    def collect(self, ticket):
        number, sampled = ticket
        assert number == self.collected + 1, "steps are collected in the order they were launched"
        self.collected = number
        return sampled

    def execute(self, entries):
        return self.collect(self.launch(entries))


def make_ahead(pages=64, **overrides):
    values = dict(max_seq_len=256, page_size=16, max_num_seqs=4, max_num_batched_tokens=64, max_chunk_size=32)
    values.update(overrides)
    config = EngineConfig(**values)
    executor = RunAheadExecutor(config, pages)
    return Scheduler(executor, config, stop_token_ids=[7]), executor


def test_running_ahead_launches_the_next_step_before_it_reads_the_previous_one():
    scheduler, executor = make_ahead()
    request = scheduler.add_request(list(range(5)), greedy(4), "a")
    scheduler.step()
    assert executor.launched == 1 and executor.collected == 0
    assert request.output_token_ids == [-1]                  # a stand-in: row 0 of the step in flight
    scheduler.step()
    assert executor.launched == 2 and executor.collected == 1
    assert request.output_token_ids == [1000, -1]
    scheduler.run_to_completion()
    assert request.output_token_ids == [1000, 1001, 1002, 1003] and request.finish_reason == "length"
    assert executor.launched == 4 and executor.collected == 4       # no step beyond the last token
    assert executor.fed[1:] == [[1000], [1001], [1002]]              # each step saw the token before it
    assert executor.cache.num_free_pages() == 64 and executor.cache.num_free_slots == 4


def test_running_ahead_gives_the_same_tokens_and_steps_as_lockstep():
    def run(ahead):
        scheduler, executor = make_ahead(run_ahead=ahead, max_num_batched_tokens=48)
        requests = [scheduler.add_request(list(range(n)), greedy(g), name)
                    for name, n, g in (("a", 40, 6), ("b", 9, 3), ("c", 70, 5), ("d", 3, 9))]
        scheduler.run_to_completion()
        return [r.output_token_ids for r in requests], executor.steps, executor
    tokens_ahead, steps_ahead, executor = run(True)
    tokens_lock, steps_lock, _ = run(False)
    assert tokens_ahead == tokens_lock
    assert steps_ahead == steps_lock
    assert all(t >= 0 for fed in executor.fed for t in fed)
    assert executor.cache.num_free_pages() == 64


def test_running_ahead_drops_the_token_of_the_step_past_a_stop_token():
    scheduler, executor = make_ahead()
    executor.stop_after["a"] = 2
    a = scheduler.add_request(list(range(5)), greedy(10), "a")
    b = scheduler.add_request(list(range(6)), greedy(5), "b")
    scheduler.run_to_completion()
    assert a.output_token_ids == [1000, 1001] and a.finish_reason == "eos"
    assert b.output_token_ids == [1000, 1001, 1002, 1003, 1004] and b.finish_reason == "length"
    # a ran one step past its stop token (the host learnt of it a step late), never two
    assert sum(1 for step in executor.steps for entry in step if entry[0] == "a") == 4
    assert executor.cache.num_free_pages() == 64 and executor.cache.num_free_slots == 4


def test_running_ahead_with_eviction_keeps_every_token():
    scheduler, executor = make_ahead(pages=5, max_seq_len=64)
    a = scheduler.add_request(list(range(30)), greedy(20), "a")
    b = scheduler.add_request(list(range(30)), greedy(20), "b")
    scheduler.run_to_completion()
    assert scheduler.num_preemptions >= 1
    for request in (a, b):
        assert request.output_token_ids == [1000 + i for i in range(20)], request.output_token_ids
    assert all(t >= 0 for fed in executor.fed for t in fed)
    assert executor.cache.num_free_pages() == 5


def test_a_repetition_penalty_keeps_the_steps_in_lockstep():
    scheduler, executor = make_ahead()
    request = scheduler.add_request(list(range(5)), SamplingParams(temperature=0.0, repetition_penalty=1.3, max_gen_len=3), "a")
    scheduler.step()
    assert executor.launched == 1 and executor.collected == 1 and request.output_token_ids == [1000]
    scheduler.run_to_completion()
    assert request.output_token_ids == [1000, 1001, 1002]


def test_abort_while_a_step_is_in_flight():
    scheduler, executor = make_ahead()
    a = scheduler.add_request(list(range(5)), greedy(10), "a")
    b = scheduler.add_request(list(range(5)), greedy(3), "b")
    scheduler.step(), scheduler.step()
    scheduler.abort(a)
    assert a.finish_reason == "abort" and all(t >= 0 for t in a.output_token_ids)
    scheduler.run_to_completion()
    assert b.output_token_ids == [1000, 1001, 1002]
    assert executor.cache.num_free_pages() == 64 and executor.cache.num_free_slots == 4


# ------------------------------------------------------------------ random workloads
@pytest.mark.parametrize("seed", range(8))
@pytest.mark.parametrize("ahead", [False, True])
def test_random_arrivals_lengths_stops_and_aborts_lose_nothing(seed, ahead):
    """Requests of random length arrive at random steps into a pool too small for all of them, some
    stop early on a stop token, some are aborted: every survivor gets exactly its tokens, the model
    never sees a stand-in id, and when all is done every page and slot is back."""
    import random

    rng = random.Random(seed)
    pages = rng.randint(9, 16)
    maker = make_ahead if ahead else make
    scheduler, executor = maker(pages=pages, max_seq_len=96, max_num_seqs=3, max_num_batched_tokens=rng.choice([24, 40, 64]),
                                max_chunk_size=rng.choice([7, 16, 32]))
    plan = []                                      # (arrival step, prompt length, tokens wanted, stop after, abort at step)
    for index in range(12):
        prompt = rng.randint(1, 60)
        wanted = rng.randint(1, 95 - prompt)
        stop = rng.randint(0, wanted) if rng.random() < 0.3 else None
        abort = rng.randint(0, 40) if rng.random() < 0.2 else None
        plan.append((rng.randint(0, 30), prompt, wanted, stop, abort))
    requests = {}
    step = 0
    while step < 400 and (len(requests) < len(plan) or scheduler.has_unfinished()):
        for index, (arrival, prompt, wanted, stop, abort) in enumerate(plan):
            if arrival == step:
                if stop is not None:
                    executor.stop_after[index] = stop
                requests[index] = scheduler.add_request([rng.randrange(100) + 10 for _ in range(prompt)], greedy(wanted), index)
            if abort == step and index in requests:
                scheduler.abort(index)
        if scheduler.has_unfinished():
            scheduler.step()
        executor.cache.check()
        step += 1
    assert len(requests) == len(plan) and not scheduler.has_unfinished()
    for index, (arrival, prompt, wanted, stop, abort) in enumerate(plan):
        request = requests[index]
        assert all(token >= 0 for token in request.output_token_ids)
        if request.finish_reason == "abort":
            continue
        count = wanted if stop is None else min(wanted, stop)
        assert request.output_token_ids == [1000 + i for i in range(count)], (index, request.finish_reason)
        assert request.finish_reason == ("eos" if stop is not None and stop < wanted else "length")
    if ahead:
        assert all(token >= 0 for fed in executor.fed for token in fed)
    assert executor.cache.num_free_pages() == pages and executor.cache.num_free_slots == 3


# ------------------------------------------------------------------ the repeat breaker
def test_the_repeat_breaker_agrees_with_the_references_own():
    """``tests/golden/repetition.json`` holds the verdicts of the reference's ``detect_repetition``
    (``rapid_llm/engine/stop_criteria.py:63-79``) on texts made by ``tests/golden/make_repetition_golden.py``."""
    import json
    from pathlib import Path

    from rapid_llm_b200.engine.repetition import text_repeats

    cases = json.loads((Path(__file__).parent / "golden" / "repetition.json").read_text())
    assert len(cases) >= 50 and 5 <= sum(case["repeats"] for case in cases) <= len(cases) - 5
    for number, case in enumerate(cases):
        assert text_repeats(case["text"]) == case["repeats"], number


def looping_text(token_ids):
    """A stand-in tokenizer: 16 characters per token, the same again every 8 tokens, so the text
    is a loop of 128 characters whatever the (all different) token ids are."""
    return "".join(f"<piece {'abcdefgh'[token % 8]} of h>. " for token in token_ids)


@pytest.mark.parametrize("ahead", [False, True])
def test_a_request_whose_text_loops_ends_with_the_reason_repeat(ahead):
    config = EngineConfig(max_seq_len=256, page_size=16, max_num_seqs=4, max_num_batched_tokens=64,
                          max_chunk_size=32, run_ahead=ahead)
    executor = RunAheadExecutor(config, 64)
    scheduler = Scheduler(executor, config, stop_token_ids=[7], detokenize=looping_text)
    assert len(looping_text([1000])) == 16
    looping = scheduler.add_request(list(range(5)), greedy(200), "loops")
    deaf = scheduler.add_request(list(range(5)), SamplingParams(temperature=0.0, repetition_penalty=1.0,
                                                                stop_on_repeat=False, max_gen_len=60), "deaf")
    scheduler.run_to_completion()
    # 512 characters (32 tokens) are the least the breaker looks at, and it looks every eighth step;
    # running ahead, a step's tokens are read one step later
    assert looping.finish_reason == "repeat"
    assert len(looping.output_token_ids) == (39 if ahead else 32)
    assert all(token >= 0 for token in looping.output_token_ids)
    assert deaf.finish_reason == "length" and len(deaf.output_token_ids) == 60
    assert executor.cache.num_free_pages() == 64 and executor.cache.num_free_slots == 4
    executor.cache.check()


def test_without_a_detokenizer_no_request_ends_for_repeating():
    scheduler, executor = make()
    request = scheduler.add_request(list(range(5)), greedy(80), "a")
    scheduler.run_to_completion()
    assert request.finish_reason == "length" and len(request.output_token_ids) == 80


def test_a_decode_bucket_stays_within_what_a_step_may_carry():
    """Padding rows of a graph-replayed decode step count as tokens: the bucket never exceeds the token
    budget (40 requests under a budget of 48 tokens pad to 48, not to 64) nor the number of slots."""
    from rapid_llm_b200.engine.runner import decode_bucket

    assert decode_bucket(40, 64, 48) == 48
    assert decode_bucket(33, 64, 8192) == 64
    assert decode_bucket(3, 64, 8192) == 4
    assert decode_bucket(5, 6, 8192) == 6
    assert decode_bucket(1, 64, 48) == 1
    for count in range(1, 49):
        assert count <= decode_bucket(count, 64, 48) <= 48


def test_a_long_request_fits_a_small_pool_of_a_windowed_group():
    """Five pages of 16 hold a window of 32 keys, a portion of 32 tokens and the ragged page at either end:
    a request of 200 tokens runs through such a pool, since the pages its window has passed come back;
    with all keys kept the same pool refuses it at submission."""
    window = [CacheNeed("window", 1, 16, window=32)]
    scheduler, executor = make(pages=5, needs=window)
    request = scheduler.add_request(list(range(190)), greedy(10), "long")
    scheduler.run_to_completion()
    assert request.finish_reason == "length" and len(request.output_token_ids) == 10
    assert executor.cache.num_free_pages() == 5
    with pytest.raises(ValueError, match="pages of cache group 0"):
        make(pages=5)[0].add_request(list(range(190)), greedy(10), "long")
    with pytest.raises(ValueError, match="pages of cache group 0"):
        make(pages=4, needs=window)[0].add_request(list(range(190)), greedy(10), "long")
