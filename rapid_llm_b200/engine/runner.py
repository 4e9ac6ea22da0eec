"""The step function: one packed batch of (request, its next tokens) through the model.

A step runs only the tokens it is given, as one batch, from the cache that earlier steps
left, and returns the logits at the wanted places.  Portions of prompts and single decoded
tokens sit side by side; a portion may be cut anywhere.  The reference runs up to three
passes of different kinds per scheduler step over padded rectangles
(``rapid_llm/engine/scheduler.py:964-988``, ``rapid_llm/executor/worker.py:339-366``); its
description of one pass is ``ModelInput`` (``rapid_llm/executor/worker.py:69-126``).

The runner owns the model, the cache (bookkeeping and device storage), the activation
workspace and the per-step metadata upload (one pinned buffer, one copy).
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Hashable, Mapping, Sequence

import numpy as np
import torch

from ..cache import CacheManager, CacheStorage, plan_groups
from ..config import EngineConfig, load_config
from ..models.causal_lm import CausalLM
from ..ops import gemm, kernels
from ..parts.base import StepShape
from ..weights import fill_random_on_device, load_weights
from .batch import GroupView, LayerCache, StepBatch, Workspace


class OutOfPages(RuntimeError):
    """A step asked for more cache pages than the pool has free."""


@dataclass
class StepEntry:
    """One request's share of a step.

    Attributes:
        request_id: Key of a request admitted with :meth:`ModelRunner.admit`.
        tokens: Its next tokens (a portion of the prompt, or one decoded token).
        want: Places among ``tokens`` whose logits are asked for; may be empty.
    """

    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


def decode_bucket(count: int, max_num_seqs: int, max_num_batched_tokens: int) -> int:
    """The next power of two from ``count`` up, but never more rows than a step may carry: the padding
    rows are tokens of the step like any other, so the bucket stays within both limits (a limit that
    is no power of two is then a bucket of its own)."""
    limit = min(max_num_seqs, max_num_batched_tokens)
    if count > limit:
        return count
    bucket = 1
    while bucket < count:
        bucket *= 2
    return min(bucket, limit)


def pages_that_fit(free_bytes: int, fraction: float, page_bytes: int, reserve: int, cap: int) -> int:
    """Cache pages for ``fraction`` of the free memory after ``reserve`` bytes are set aside for the
    largest step's activations and logits; never more than ``cap`` (what the slots can hold at full
    length), never fewer than one."""
    usable = int(free_bytes * fraction) - int(reserve)
    pages = usable // page_bytes if page_bytes > 0 else cap
    return int(max(1, min(pages, cap)))


def require_cuda(device: torch.device) -> None:
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError(
            "rapid_llm_b200 runs on an NVIDIA B200 through its own CUDA kernels; "
            f"no CUDA device is available for {device} and there is no CPU path"
        )


class ModelRunner:
    def __init__(self, model: CausalLM, config: EngineConfig, *, num_pages: int | None = None) -> None:
        require_cuda(model.device)
        if model.dtype != config.dtype:
            raise ValueError(f"model dtype {model.dtype} differs from the engine's {config.dtype}")
        self.model = model
        self.config = config
        self.device = model.device
        self.dtype = model.dtype
        if config.max_seq_len > model.spec.max_positions:
            raise ValueError(
                f"max_seq_len ({config.max_seq_len}) exceeds the model's max positions "
                f"({model.spec.max_positions})"
            )
        groups, self.entry_group = plan_groups(model.cache_needs())
        pages = num_pages if num_pages is not None else config.num_pages
        if pages is None:
            pages = self._pages_from_free_memory(groups)
        self.cache = CacheManager(
            groups,
            page_size=config.page_size,
            num_pages=pages,
            max_num_seqs=config.max_num_seqs,
            max_seq_len=config.max_seq_len,
            extra_table_rows=1,  # an all-null row: the slot of a captured decode batch's padding
        )
        self.pad_slot = config.max_num_seqs
        self.storage = CacheStorage(self.cache, self.entry_group, model.state_needs(), self.dtype, self.device)
        self.workspace = Workspace(config.max_num_batched_tokens, self.device)

        t_max, n_max, g = config.max_num_batched_tokens, config.max_num_seqs + 1, len(groups)
        self._planners = model.step_planners()
        self._meta_capacity = t_max * (4 + g) + 3 * n_max + 8 + sum(
            planner.capacity(t_max, n_max) + 8 for planner in self._planners
        ) + g * (n_max * (config.max_pages_per_seq + 1) + 8)      # block-table rows that changed
        self._meta_host = [
            torch.empty(self._meta_capacity, dtype=torch.int32, pin_memory=True) for _ in range(2)
        ]
        # a host buffer is written again only after the copy that last read it has run: steps that
        # sample nothing are never waited for, so the host can be many steps ahead of the device
        self._meta_copied: list[torch.cuda.Event | None] = [None, None]
        self._meta_flip = 0
        self._meta_device = torch.zeros(self._meta_capacity, dtype=torch.int32, device=self.device)
        # word 0: the kernels' fault word; words 1..: the step's sampled tokens (one read brings both)
        self.result = torch.zeros(config.max_num_seqs + 2, dtype=torch.int32, device=self.device)
        self.fault = self.result[:1]
        self.steps_run = 0
        self._graphs: dict[tuple, tuple[torch.cuda.CUDAGraph, torch.Tensor, int]] = {}      # by (bucket, launch constants)
        self._graph_pool = None

    # -- construction ---------------------------------------------------------------- #
    @classmethod
    def from_folder(
        cls, model_dir: str | Path, config: EngineConfig, overrides: Mapping[str, Any] | None = None,
        device: str | torch.device = "cuda:0", num_pages: int | None = None,
    ) -> "ModelRunner":
        """Build the model named by the folder's ``config.json`` and load its safetensors."""
        device = torch.device(device)
        require_cuda(device)
        model_config = load_config(model_dir, overrides)
        model = CausalLM(model_config.to_spec(), config.dtype, device)
        load_weights(model, model_dir)
        runner = cls(model, config, num_pages=num_pages)
        runner.model_config = model_config
        return runner

    @classmethod
    def from_random(
        cls, model_config, seed: int, config: EngineConfig, device: str | torch.device = "cuda:0",
        num_pages: int | None = None, std: float = 0.02, norm_std: float = 0.0,
    ) -> "ModelRunner":
        """A model of the given configuration with weights drawn on the device."""
        device = torch.device(device)
        require_cuda(device)
        model = CausalLM(model_config.to_spec(), config.dtype, device)
        fill_random_on_device(model, seed, std=std, norm_std=norm_std)
        runner = cls(model, config, num_pages=num_pages)
        runner.model_config = model_config
        return runner

    def _pages_from_free_memory(self, groups) -> int:
        free, _total = torch.cuda.mem_get_info(self.device)
        element = torch.empty((), dtype=self.dtype).element_size()
        per_page = sum(len(g.entries) * g.need.elements_per_token() * self.config.page_size * element for g in groups)
        return pages_that_fit(
            free, self.config.memory_fraction, per_page,
            reserve=self.config.max_num_batched_tokens * self.model.activation_bytes_per_token()
            + self.config.max_num_seqs * self.model.spec.vocab_size * (element + 4),
            cap=self.config.max_num_seqs * self.config.max_pages_per_seq,
        )

    # -- life of a request -------------------------------------------------------------- #
    def admit(self, request_id: Hashable) -> bool:
        slot = self.cache.admit(request_id)
        if slot is None:
            return False
        self.storage.reset_state(slot)
        return True

    def release(self, request_id: Hashable) -> None:
        self.cache.release(request_id)

    def num_cached_tokens(self, request_id: Hashable) -> int:
        return self.cache.num_tokens(request_id)

    # -- the step ----------------------------------------------------------------------- #
    def prepare(self, entries: Sequence[StepEntry], pad_to: int | None = None) -> StepBatch:
        """Reserve pages, lay the step's metadata out and upload it."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        cache, config = self.cache, self.config
        lengths = [len(entry.tokens) for entry in entries]
        if min(lengths) < 1:
            raise ValueError("an entry carries no tokens")
        total = sum(lengths)
        pad = 0 if pad_to is None else pad_to - len(entries)
        if pad < 0 or (pad and max(lengths) != 1):
            raise ValueError("only single-token steps can be padded")
        n, t = len(entries) + pad, total + pad
        if t > config.max_num_batched_tokens:
            raise ValueError(f"step of {t} tokens exceeds max_num_batched_tokens {config.max_num_batched_tokens}")
        if len({entry.request_id for entry in entries}) != len(entries):
            raise ValueError("a request appears twice in one step")
        for entry, length in zip(entries, lengths):      # refuse before any page is taken
            for place in entry.want:
                if not 0 <= place < length:
                    raise ValueError(f"want index {place} outside the entry's {length} tokens")

        starts = [cache.num_tokens(entry.request_id) for entry in entries]
        short = [
            entry.request_id
            for entry, start, length in zip(entries, starts, lengths)
            if start + length > config.max_seq_len
        ]
        if short:
            raise ValueError(f"requests {short} would exceed max_seq_len {config.max_seq_len}")
        for index, pool in enumerate(cache.pools):
            needed = sum(
                cache.pages_needed(entry.request_id, start + length)[index]
                for entry, start, length in zip(entries, starts, lengths)
            )
            if needed > pool.num_free:
                raise OutOfPages(
                    f"the step needs {needed} pages of cache group {index}, {pool.num_free} are free"
                )
        for entry, start, length in zip(entries, starts, lengths):
            reserved = cache.reserve(entry.request_id, start + length)
            assert reserved

        g = len(cache.groups)
        rows = sum(len(entry.want) for entry in entries) + pad
        flip = self._meta_flip
        host = self._meta_host[flip]
        self._meta_flip ^= 1
        if self._meta_copied[flip] is not None:
            self._meta_copied[flip].synchronize()
        meta = host.numpy()
        offsets: dict[str, tuple[int, int]] = {}
        cursor = 0

        def carve(name: str, count: int) -> np.ndarray:
            nonlocal cursor
            offsets[name] = (cursor, count)
            view = meta[cursor : cursor + count]
            cursor += count
            return view

        token_ids, positions, token_slot = carve("token_ids", t), carve("positions", t), carve("token_slot", t)
        cu_seqlens, entry_slot, entry_start = carve("cu_seqlens", n + 1), carve("entry_slot", n), carve("entry_start", n)
        kv_dest = [carve(f"kv_dest{i}", t) for i in range(g)]
        logit_rows = carve("logit_rows", rows)
        shape = StepShape(
            lengths=np.asarray(lengths + [1] * pad, dtype=np.int32),
            starts=np.asarray(starts + [0] * pad, dtype=np.int32),
            decode_only=max(lengths) == 1,
            page_size=cache.page_size,
            padding=pad,
        )
        planned: dict[tuple, dict[str, Any]] = {}
        for planner in self._planners:
            plan = planner.plan(shape)
            for name, value in plan.items():
                if isinstance(value, np.ndarray):
                    cursor = -(-cursor // 4) * 4          # 16-byte aligned arrays
                    carve(f"plan:{planner.key}:{name}", value.size)[:] = value.reshape(-1)
            planned[planner.key] = plan
        if cursor > self._meta_capacity:
            raise ValueError("the step's metadata does not fit its buffer")

        at, row_at = 0, 0
        cu_seqlens[0] = 0
        for i, (entry, start, length) in enumerate(zip(entries, starts, lengths)):
            slot = cache.slot_of(entry.request_id)
            token_ids[at : at + length] = np.asarray(entry.tokens, dtype=np.int64).astype(np.int32)
            positions[at : at + length] = np.arange(start, start + length, dtype=np.int32)
            token_slot[at : at + length] = slot
            entry_slot[i], entry_start[i] = slot, start
            for index in range(g):
                kv_dest[index][at : at + length] = cache.kv_destinations(index, slot, start, length)
            for place in entry.want:
                logit_rows[row_at] = at + place
                row_at += 1
            at += length
            cu_seqlens[i + 1] = at
        for i in range(len(entries), n):  # padding rows of a captured decode batch
            token_ids[at], positions[at], token_slot[at] = 0, 0, self.pad_slot
            entry_slot[i], entry_start[i] = self.pad_slot, 0
            for index in range(g):
                kv_dest[index][at] = 0
            logit_rows[row_at] = at
            row_at += 1
            at += 1
            cu_seqlens[i + 1] = at

        # block-table rows that changed on the host ride along and are put in place by a kernel
        changed: list[tuple[int, str, str]] = []
        for index in range(g):
            slots = cache.take_dirty(index)
            if not slots:
                continue
            table = cache.block_tables[index]
            cursor = -(-cursor // 4) * 4
            carve(f"table_slots{index}", len(slots))[:] = slots
            carve(f"table_rows{index}", len(slots) * table.shape[1])[:] = table[slots].reshape(-1)
            changed.append((index, f"table_slots{index}", f"table_rows{index}"))
        if cursor > self._meta_capacity:
            raise ValueError("the step's metadata does not fit its buffer")
        self._meta_device[:cursor].copy_(host[:cursor], non_blocking=True)
        if self._meta_copied[flip] is None:
            self._meta_copied[flip] = torch.cuda.Event()
        self._meta_copied[flip].record()

        def dev(name: str) -> torch.Tensor:
            begin, count = offsets[name]
            return self._meta_device[begin : begin + count]

        for index, slots_name, rows_name in changed:
            kernels.scatter_rows(self.storage.block_tables[index], dev(slots_name), dev(rows_name), self.fault)

        extras = {
            key: {
                name: dev(f"plan:{key}:{name}").view(value.shape) if isinstance(value, np.ndarray) else value
                for name, value in plan.items()
            }
            for key, plan in planned.items()
        }
        ends = [start + length for start, length in zip(starts, lengths)]
        views = [
            GroupView(
                block_table=self.storage.block_tables[index],
                kv_dest=dev(f"kv_dest{index}"),
                page_size=cache.page_size,
                window=cache.groups[index].window,
            )
            for index in range(g)
        ]
        return StepBatch(
            num_tokens=t,
            num_entries=n,
            token_ids=dev("token_ids"),
            positions=dev("positions"),
            token_slot=dev("token_slot"),
            cu_seqlens=dev("cu_seqlens"),
            entry_slot=dev("entry_slot"),
            entry_start=dev("entry_start"),
            logit_rows=dev("logit_rows"),
            h_cu_seqlens=cu_seqlens.copy(),
            h_entry_slot=entry_slot.copy(),
            h_entry_start=entry_start.copy(),
            max_query_len=max(lengths),
            max_context_len=max(ends),
            groups=views,
            workspace=self.workspace,
            fault=self.fault,
            dtype=self.dtype,
            decode_only=max(lengths) == 1,
            extras=extras,
            feedback=self.result[1:],
        )

    def layer_caches(self) -> list[LayerCache]:
        caches = []
        for position, entry in enumerate(self.model.spec.schedule):
            group, pages = self.storage.entry_pages(position, entry.cache_from)
            state = self.storage.states[position]
            caches.append(LayerCache(group=group, pages=pages, writes=entry.cache_from is None, state=state))
        return caches

    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the entries as one batch; logits ``[wanted, vocab]`` in entry and ``want`` order."""
        batch = self.prepare(entries)
        logits = self._forward(batch, self.layer_caches())
        for entry in entries:
            self.cache.release_passed(entry.request_id)
        self.steps_run += 1
        return logits

    def _forward(self, batch: StepBatch, caches: list[LayerCache]) -> torch.Tensor:
        """The model over one batch, its kernels chained by programmatic dependent launch if configured."""
        previous = kernels.PDL
        kernels.PDL = self.config.use_dependent_launch
        try:
            logits = self.model.forward(batch, caches)
            gemm.flush()         # products still queued for the persistent kernel (a step that wants no logits)
            return logits
        finally:
            kernels.PDL = previous

    def decode_bucket(self, count: int) -> int:
        """Batch size a decode-only step of ``count`` rows is padded to for graph replay."""
        return decode_bucket(count, self.config.max_num_seqs, self.config.max_num_batched_tokens)

    @torch.no_grad()
    def step_decode(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """A step of single tokens, each wanting its logits, replayed from a captured graph.

        The batch is padded to a bucket size with rows that point at the null page; the
        metadata lives in a fixed device buffer that is refreshed before each replay.  The
        first step of a bucket (and of a set of the planners' launch constants, which change at a few
        context lengths) runs eagerly and is then captured.  The reference captures
        decode graphs per batch size and length bucket (``rapid_llm/executor/cuda_graph.py:45-46,317``).
        """
        if any(len(entry.tokens) != 1 or list(entry.want) != [0] for entry in entries):
            raise ValueError("step_decode takes single tokens that all want their logits")
        count = len(entries)
        bucket = self.decode_bucket(count)
        batch = self.prepare(entries, pad_to=bucket)
        # what a captured step has baked in beside its addresses: the bucket and the planners' launch constants
        # (plain values and the sizes of their lists); a step that differs in one of them is another graph
        constants = tuple(
            (str(key), name, tuple(value.shape) if isinstance(value, torch.Tensor)
             else value if isinstance(value, (int, float, bool, str, type(None))) else repr(value))
            for key, plan in sorted(batch.extras.items(), key=lambda item: str(item[0])) for name, value in sorted(plan.items())
        )
        graph_key = (bucket, constants)
        captured = self._graphs.get(graph_key)
        if captured is None:
            caches = self.layer_caches()
            logits = self._forward(batch, caches)
            graph = torch.cuda.CUDAGraph()
            torch.cuda.synchronize(self.device)
            before = kernels.LAUNCHES.count
            with torch.cuda.graph(graph, pool=self._graph_pool):
                static_logits = self._forward(batch, caches)
            launches = kernels.LAUNCHES.count - before
            kernels.LAUNCHES.count = before          # recording is not launching
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            # The eager run above is this step's result.  Capturing executes nothing, and the graph
            # is not replayed now: a mixer with state of its own must see every token once.
            self._graphs[graph_key] = (graph, static_logits, launches)
        else:
            graph, logits, launches = captured
            graph.replay()
            kernels.LAUNCHES.add(launches)
        for entry in entries:
            self.cache.release_passed(entry.request_id)
        self.steps_run += 1
        return logits[:count]

    def check_fault(self) -> None:
        """Raise if a kernel met an index outside its tables since the last check (syncs)."""
        word = int(self.fault.item())
        if word:
            self.fault.zero_()
            kernels.gemm_chain_reset(self.device)      # a kernel that gave up leaves its counters as they were
            raise RuntimeError(f"a kernel reported a fault: {kernels.describe_fault(word)}")

    def memory_report(self) -> dict[str, int]:
        return {
            "weights": self.model.parameter_bytes(),
            "cache": self.storage.nbytes(),
            "workspace": self.workspace.nbytes(),
        }
