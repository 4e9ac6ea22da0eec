"""Continuous batching above the step function: admit, cut prompts, decode, finish, free.

Each call of :meth:`Scheduler.step` plans ONE packed batch under a token budget: the next
token of every request that is decoding, then the next portion of every prompt that is
under way, then new admissions in arrival order; runs it; harvests the sampled tokens;
finishes and frees.  The policy is the reference's (``rapid_llm/engine/batch_planner.py:
462-523,579-666,683-698``), with the budget counted in real tokens instead of a padded
rectangle, and one pass per step instead of up to three (``rapid_llm/engine/scheduler.py:964-988``).

When pages run out:

* a waiting request stays waiting (admission never evicts);
* a running request that cannot grow evicts the *youngest* running request, which gives
  back its pages, folds the tokens it has generated into its prompt and goes to the front
  of the queue to be recomputed (``rapid_llm/engine/batch_planner.py:849-888,972-1023``);
  if the request that cannot grow is itself the youngest, it is the one evicted;
* with eviction off, it waits for others to finish; if every running request is stuck,
  :class:`CacheExhausted` is raised rather than spinning;
* a request that could never fit the pool even alone is refused when it is submitted.

A request ends with ``"eos"`` (a stop token, which is not appended), ``"length"``, ``"abort"`` or,
when the scheduler was given a detokenizer, ``"repeat"``: every eighth step the text of a request
with ``stop_on_repeat`` is checked for a loop (``engine/repetition.py``), as the reference does
(``rapid_llm/engine/scheduler.py:1398-1455``).

Running ahead.  A step's sampled tokens stay on the device, where the next step's embedding
can pick them up, so the next step can be planned and enqueued before the host has seen them:
everything else a step needs (positions, pages, which rows to sample) follows from counts.
With ``run_ahead`` the scheduler therefore enqueues step N+1 and only then reads step N's
tokens, while the GPU is already busy; a token that is known only on the device stands in
the request's list as the negative number ``-(row + 1)`` of its row in the previous step's
result.  What the host learns one step late is a stop token: the token that the request's
extra step produced is dropped.  The reference runs the same launch/harvest pipeline with
device-side token feedback (``rapid_llm/engine/scheduler.py:817-933``).  Requests with a
repetition penalty need their tokens on the host for the next step and are stepped in
lockstep instead.
"""

from __future__ import annotations

import itertools
import time
import zlib
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Hashable, Protocol, Sequence

from ..cache import CacheManager
from ..config import EngineConfig
from ..sampling.params import SamplingParams
from .repetition import CHECK_EVERY, text_repeats

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


class CacheExhausted(RuntimeError):
    """No running request can make progress and eviction is off."""


@dataclass
class Request:
    """One generation request; token ids in, token ids out."""

    request_id: Hashable
    prompt_token_ids: list[int]
    params: SamplingParams
    max_new_tokens: int
    seed: int
    status: str = WAITING
    output_token_ids: list[int] = field(default_factory=list)
    num_computed_tokens: int = 0
    finish_reason: str | None = None
    num_preemptions: int = 0
    exhausted: bool = False        # its last token is sampled (perhaps still on the device): nothing more to feed
    arrival_time: float = 0.0
    first_scheduled_time: float | None = None
    first_token_time: float | None = None
    finish_time: float | None = None

    @property
    def all_token_ids(self) -> list[int]:
        return self.prompt_token_ids + self.output_token_ids

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def finished(self) -> bool:
        return self.status == FINISHED


@dataclass
class PlannedEntry:
    """A request's share of the planned step; ``samples`` = its last token is fed, so the
    step's logits there choose its next token."""

    request: Request
    start: int
    tokens: list[int]
    samples: bool


@dataclass
class Inflight:
    """A step that is enqueued but whose sampled tokens the host has not read yet."""

    entries: list[PlannedEntry]
    handle: object
    slots: list[tuple[Request, int]]    # per sampled row: the request and the index of its stand-in token


@dataclass
class StepPlan:
    entries: list[PlannedEntry] = field(default_factory=list)
    preempted: list[Request] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(len(entry.tokens) for entry in self.entries)


class Executor(Protocol):
    """What the scheduler needs below it; the device executor and the tests' fake provide it."""

    cache: CacheManager

    def admit(self, request_id: Hashable) -> bool: ...

    def release(self, request_id: Hashable) -> None: ...

    def execute(self, entries: Sequence[PlannedEntry]) -> list[int]:
        """Run the entries as one batch; one sampled token per entry with ``samples`` set, in order.

        An executor that can run ahead also has ``launch(entries) -> handle`` (enqueue only) and
        ``collect(handle) -> list[int]`` (wait for that step's tokens); a token id ``-(row + 1)``
        among the entries' tokens then means row ``row`` of the previously launched step's result."""


class Scheduler:
    def __init__(self, executor: Executor, config: EngineConfig, stop_token_ids: Sequence[int] = (),
                 detokenize: Callable[[list[int]], str] | None = None) -> None:
        """``detokenize`` (token ids to text) switches the repeat breaker on for requests with
        ``stop_on_repeat``; without it no request ends with the reason ``"repeat"``."""
        self.executor = executor
        self.detokenize = detokenize
        self.cache = executor.cache
        self.config = config
        self.stop_token_ids = set(int(t) for t in stop_token_ids)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []      # in admission order: the last is the youngest
        self._ids = itertools.count()
        self.num_steps = 0
        self.num_preemptions = 0
        self._inflight: Inflight | None = None
        self._can_launch = hasattr(executor, "launch") and hasattr(executor, "collect")

    @classmethod
    def from_pretrained(cls, model, **options) -> "Scheduler":
        """A scheduler over a model folder, as the reference builds one
        (``rapid_llm/engine/scheduler.py:410-440``): the options are those of
        :class:`~rapid_llm_b200.engine.llm.LLM` (``max_seq_len``, ``max_num_seqs``,
        ``max_num_batched_tokens``, ``max_chunk_size``, ``max_gpu_num_blocks``, ``use_cuda_graph``,
        ``enable_preemption``, ``hf_overrides``, ``dtype``, ...).  The entry point it was built
        through stays reachable as ``scheduler.llm``."""
        from .llm import LLM

        llm = LLM(model, **options)
        llm.scheduler.llm = llm
        return llm.scheduler

    # -- submission ------------------------------------------------------------------ #
    def add_request(
        self,
        prompt: Sequence[int] | str,
        params: SamplingParams | None = None,
        request_id: Hashable | None = None,
        prompt_token_ids: Sequence[int] | None = None,
        sampling_params: SamplingParams | None = None,
    ) -> Request:
        """Queue a request.  An empty prompt, or one that leaves no room to generate, is refused
        (``rapid_llm/engine/batch_planner.py:403-427``); so is one the pool could never hold.

        ``prompt`` is the list of token ids.  The reference's calling form, text first and the
        ids in ``prompt_token_ids`` (``rapid_llm/engine/scheduler.py:635-643``), is taken too: the
        ids win, and text without ids is refused, since the scheduler holds no tokenizer
        (``LLM.generate`` encodes text).  ``sampling_params`` is the reference's name of ``params``."""
        params = params or sampling_params or SamplingParams()
        if prompt_token_ids is not None:
            prompt = prompt_token_ids
        elif isinstance(prompt, str):
            raise ValueError("the scheduler takes token ids: pass prompt_token_ids, or use LLM.generate for text")
        prompt = [int(t) for t in prompt]
        limit = self.config.max_seq_len
        if not prompt:
            raise ValueError("the prompt is empty")
        if len(prompt) >= limit:
            raise ValueError(f"the prompt has {len(prompt)} tokens, max_seq_len is {limit}")
        room = limit - len(prompt)
        max_new = min(params.max_gen_len or room, room)
        page = self.cache.page_size
        most = len(prompt) + max_new - 1          # tokens cached when the last one is sampled
        # the largest portion of it a step can carry; a windowed group holds at most its window, that
        # portion and the ragged page at either end at a time, since passed pages are given back
        portion = min(self.config.max_chunk_size, self.config.max_num_batched_tokens) if self.config.enable_chunked_prefill else len(prompt)
        for index, pool in enumerate(self.cache.pools):
            window = self.cache.groups[index].window
            pages = -(-most // page)
            if window:
                pages = min(pages, -(-(window + portion) // page) + 1)
            if pages > pool.num_pages:
                raise ValueError(
                    f"the request needs {pages} pages of cache group {index} by itself, "
                    f"the pool has {pool.num_pages}"
                )
        if request_id is None:
            request_id = f"req-{next(self._ids)}"
        seed = params.seed if params.seed is not None else zlib.crc32(repr(request_id).encode())
        request = Request(request_id, prompt, params, max_new, seed, arrival_time=time.perf_counter())
        self.waiting.append(request)
        return request

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running or self._inflight is not None)

    has_unfinished_requests = has_unfinished      # the reference's name

    # -- planning -------------------------------------------------------------------- #
    def _chunk(self, request: Request, budget: int) -> int:
        remaining = request.num_tokens - request.num_computed_tokens
        if self.config.enable_chunked_prefill:
            return min(remaining, self.config.max_chunk_size, budget)
        return remaining if remaining <= budget else 0

    def _fits(self, request: Request, upto: int, free: list[int]) -> list[int] | None:
        """Pages per group the growth takes, or ``None`` if some pool is short."""
        if self.cache.has(request.request_id):
            needed = self.cache.pages_needed(request.request_id, upto)
        else:
            needed = [-(-upto // self.cache.page_size)] * len(self.cache.pools)
        if any(n > f for n, f in zip(needed, free)):
            return None
        return needed

    def _preempt(self, victim: Request, plan: StepPlan, free: list[int]) -> None:
        """Evict: pages back to the pool, generated tokens kept, recompute from the start."""
        before = [pool.num_free for pool in self.cache.pools]
        self.executor.release(victim.request_id)
        for index, pool in enumerate(self.cache.pools):
            free[index] += pool.num_free - before[index]
        self.running.remove(victim)
        victim.status = WAITING
        victim.num_computed_tokens = 0
        victim.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(victim)
        plan.preempted.append(victim)

    def plan(self) -> StepPlan:
        plan = StepPlan()
        budget = self.config.max_num_batched_tokens
        free = [pool.num_free for pool in self.cache.pools]
        planned: set[Hashable] = set()

        # running requests, oldest first: single decoded tokens and resumed portions
        decoding = [r for r in self.running if not r.exhausted and r.num_tokens - r.num_computed_tokens == 1]
        resumed = [r for r in self.running if not r.exhausted and r.num_tokens - r.num_computed_tokens > 1]
        for request in decoding + resumed:
            if request not in self.running:        # evicted while planning an older one
                continue
            while True:
                size = self._chunk(request, budget)
                if size <= 0:
                    break
                needed = self._fits(request, request.num_computed_tokens + size, free)
                if needed is not None:
                    self._take(plan, request, size, needed, free, planned)
                    budget -= size
                    break
                if not self.config.enable_preemption:
                    break
                victim = next(
                    (r for r in reversed(self.running) if r.request_id not in planned), None
                )
                if victim is None:
                    break
                self._preempt(victim, plan, free)
                if victim is request:
                    break

        # admissions in arrival order; the queue never skips ahead
        while self.waiting and budget > 0 and len(self.running) < self.config.max_num_seqs:
            request = self.waiting[0]
            if request in plan.preempted:
                # evicted this very step: it waits one step, and so does everyone behind it, since it
                # stands at the head of the queue and the queue never skips ahead
                break
            size = self._chunk(request, budget)
            if size <= 0 or self.cache.num_free_slots == 0:
                break
            needed = self._fits(request, size, free)
            if needed is None:
                break
            if not self.executor.admit(request.request_id):
                break
            self.waiting.popleft()
            request.status = RUNNING
            request.num_computed_tokens = 0
            if request.first_scheduled_time is None:
                request.first_scheduled_time = time.perf_counter()
            self.running.append(request)
            self._take(plan, request, size, needed, free, planned)
            budget -= size

        stuck = [r for r in self.running if not r.exhausted]
        if not plan.entries and stuck and not plan.preempted and self._inflight is None:
            raise CacheExhausted(
                f"{len(stuck)} running requests, none can grow: the cache pool "
                f"({[pool.num_pages for pool in self.cache.pools]} pages) is exhausted and eviction is off"
            )
        return plan

    def _take(self, plan, request, size, needed, free, planned) -> None:
        start = request.num_computed_tokens
        tokens = request.all_token_ids[start : start + size]
        plan.entries.append(PlannedEntry(request, start, tokens, samples=start + size == request.num_tokens))
        for index, count in enumerate(needed):
            free[index] -= count
        planned.add(request.request_id)

    # -- one step -------------------------------------------------------------------- #
    def _runs_ahead(self) -> bool:
        if not (self.config.run_ahead and self._can_launch):
            return False
        return all(r.params.repetition_penalty == 1.0 for r in itertools.chain(self.running, self.waiting))

    def _launch(self, plan: StepPlan) -> Inflight:
        """Enqueue the planned batch; every sampled row leaves a stand-in token in its request."""
        if self._can_launch:
            handle = self.executor.launch(plan.entries)
        else:
            handle = self.executor.execute(plan.entries)
        slots: list[tuple[Request, int]] = []
        for entry in plan.entries:
            request = entry.request
            request.num_computed_tokens = entry.start + len(entry.tokens)
            if not entry.samples:
                continue
            request.output_token_ids.append(-(len(slots) + 1))
            slots.append((request, len(request.output_token_ids) - 1))
            if len(request.output_token_ids) >= request.max_new_tokens or request.num_tokens >= self.config.max_seq_len:
                request.exhausted = True
        return Inflight(plan.entries, handle, slots)

    def _harvest(self, inflight: Inflight) -> list[Request]:
        """Read a launched step's tokens; put them in place of their stand-ins, finish and free."""
        sampled = self.executor.collect(inflight.handle) if self._can_launch else inflight.handle
        now = time.perf_counter()
        look_for_loops = self.detokenize is not None and self.num_steps % CHECK_EVERY == 0
        finished: list[Request] = []
        for (request, index), token in zip(inflight.slots, sampled):
            if request.finished:
                continue                                  # a step it ran ahead into: the token is dropped
            token = int(token)
            if request.first_token_time is None:
                request.first_token_time = now
            if token in self.stop_token_ids:
                del request.output_token_ids[index:]      # the stop token is not appended
                self._finish(request, "eos", now)
            else:
                request.output_token_ids[index] = token
                if request.exhausted and index == len(request.output_token_ids) - 1:
                    self._finish(request, "length", now)
                elif look_for_loops and request.params.stop_on_repeat and text_repeats(
                    self.detokenize(request.output_token_ids[: index + 1])
                ):
                    self._finish(request, "repeat", now)      # stand-ins of steps run ahead are dropped
            if request.finished:
                finished.append(request)
        return finished

    def step(self) -> list[Request]:
        """Plan and enqueue one batch and harvest one; returns the requests that finished.

        Running ahead, the batch harvested is the one enqueued by the previous call (so the
        GPU works on the new batch while the host reads the old one's tokens); otherwise it is
        the batch this call enqueued."""
        finished: list[Request] = []
        previous, self._inflight = self._inflight, None
        ahead = self._runs_ahead()
        if previous is not None and not ahead:
            finished += self._harvest(previous)
            previous = None
        self._inflight = previous          # planning may ask whether anything is still in flight
        plan = self.plan()
        self._inflight = None
        self.num_steps += 1
        current = self._launch(plan) if plan.entries else None
        if previous is not None:
            finished += self._harvest(previous)
        if current is not None and not ahead:
            finished += self._harvest(current)
            current = None
        self._inflight = current
        return finished

    def _finish(self, request: Request, reason: str, now: float) -> None:
        was_running = request.status == RUNNING
        request.status = FINISHED
        request.finish_reason = reason
        request.finish_time = now
        while request.output_token_ids and request.output_token_ids[-1] < 0:
            request.output_token_ids.pop()               # stand-ins of steps it ran ahead into
        if was_running:
            self.running.remove(request)
            self.executor.release(request.request_id)
        elif request in self.waiting:                    # evicted while its last token was in flight
            self.waiting.remove(request)

    def abort(self, request: Request | Hashable) -> None:
        """End a request now; takes the handle or, as the reference does, its id."""
        if not isinstance(request, Request):
            request = next((r for r in [*self.running, *self.waiting] if r.request_id == request), None)
            if request is None:
                return
        if request.status in (RUNNING, WAITING):
            self._finish(request, "abort", time.perf_counter())

    def run_to_completion(self) -> None:
        while self.has_unfinished():
            self.step()
