"""The generation loop: requests in, token ids out, over the step function.

Requests are run in batches that start together: each batch's prompts (of
unequal lengths) go through one step, then every live request advances by one
token per step.  A request ends at a stop token, at `max_new_tokens`, or when
it fills the model's positions; it leaves its batch at once, its slot goes
back to the cache, and the batch's later steps are smaller.  No request joins
a batch that has started; when a batch is done the next requests form the
next one, as often as needed.

Upstream runs one prompt for a fixed 601 steps, greedy, with no stop token
(inference.cpp:137-168).  This module decides on the host only; it needs a
*stepper* (alloc_slot, free_slot, step) and a *picker* (logits -> tokens),
which the GPU engine provides and which tests can fake.

When the stepper can take a step's tokens from the device (`step_decode_device`) and a
`device_picker` leaves the chosen tokens there, the loop runs one step ahead of itself: step t + 1 is
launched on the tokens of step t before the host has read them, so the GPU never waits for the host's
bookkeeping.  The decisions are the same; only a request that ends at a stop token has already been
taken one step further, and that step's token for it is dropped (its row changes nobody else's).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

from ..cache.paged import TOKEN_UNIT
from .step import StepEntry


class GenerationError(ValueError):
    pass


@dataclass(frozen=True)
class GenParams:
    max_new_tokens: int = 128
    temperature: float = 0.0          # 0 = greedy
    seed: int = 0
    stop_token_ids: tuple = ()

    def __post_init__(self):
        if self.max_new_tokens < 0:
            raise GenerationError(f"max_new_tokens must not be negative, found {self.max_new_tokens}")
        if self.temperature < 0:
            raise GenerationError(f"temperature must not be negative, found {self.temperature}")
        object.__setattr__(self, "stop_token_ids", tuple(int(t) for t in self.stop_token_ids))


@dataclass
class GenStats:
    batches: int = 0
    steps: int = 0
    prompt_tokens: int = 0
    new_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    batch_sizes: list = field(default_factory=list)     # live requests at each step
    step_times: list = field(default_factory=list)      # host clock (perf_counter) when each step's tokens had arrived


def tokens_held(prompt_len: int, max_new_tokens: int, max_positions: int) -> int:
    """Most cache positions the request can come to hold, in whole units of 64."""
    most = min(prompt_len + max(max_new_tokens - 1, 0), max_positions)
    return -(-most // TOKEN_UNIT) * TOKEN_UNIT


def plan_batches(prompt_lens: Sequence[int], max_new_tokens: int, capacity_tokens: int, max_positions: int,
                 max_batch: int) -> list[list[int]]:
    """Requests in their given order, cut into batches that fit the cache and `max_batch`."""
    batches, cur, used = [], [], 0
    for i, n in enumerate(prompt_lens):
        if n <= 0:
            raise GenerationError(f"request {i} has an empty prompt")
        if n > max_positions:
            raise GenerationError(f"request {i} has {n} prompt tokens; the model takes {max_positions} positions")
        need = tokens_held(n, max_new_tokens, max_positions)
        if need > capacity_tokens:
            raise GenerationError(f"request {i} may hold {need} tokens; the cache was sized for {capacity_tokens}")
        if cur and (used + need > capacity_tokens or len(cur) >= max_batch):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


def finished(token: int, n_new: int, prompt_len: int, params: GenParams, max_positions: int) -> bool:
    return (token in params.stop_token_ids or n_new >= params.max_new_tokens
            or prompt_len + n_new >= max_positions)


class GenerationLoop:
    def __init__(self, stepper, picker: Callable, capacity_tokens: int, max_positions: int, max_batch: int,
                 device_picker: Optional[Callable] = None):
        self.stepper, self.picker = stepper, picker
        # device_picker(logits, request ids, token indices, params) -> tokens on the device, with
        # .to_host() -> list[int]; the loop then runs one step ahead (see the module's text)
        self.device_picker = device_picker if hasattr(stepper, "step_decode_device") else None
        self.capacity_tokens, self.max_positions, self.max_batch = capacity_tokens, max_positions, max_batch
        self.stats = GenStats()

    def run(self, prompts: Sequence[Sequence[int]], params: GenParams) -> list[list[int]]:
        """Generated ids per prompt (a stop token, when met, is the last one)."""
        self.stats = GenStats()
        out: list[list[int]] = [[] for _ in prompts]
        if params.max_new_tokens == 0 or not prompts:
            return out
        for batch in plan_batches([len(p) for p in prompts], params.max_new_tokens, self.capacity_tokens,
                                  self.max_positions, self.max_batch):
            self._run_batch(batch, prompts, params, out)
        return out

    def _run_batch(self, batch: list[int], prompts, params: GenParams, out: list[list[int]]) -> None:
        if self.device_picker is not None:
            return self._run_batch_ahead(batch, prompts, params, out)
        st = self.stats
        st.batches += 1
        slot = {}
        try:
            for i in batch:
                slot[i] = self.stepper.alloc_slot()
            t0 = time.perf_counter()
            live = list(batch)
            logits = self.stepper.step([StepEntry(slot[i], list(prompts[i]), [len(prompts[i]) - 1]) for i in live])
            tokens = self.picker(logits, live, [0] * len(live), params)
            st.prefill_seconds += time.perf_counter() - t0
            st.prompt_tokens += sum(len(prompts[i]) for i in live)
            t0 = time.perf_counter()
            while True:
                st.steps += 1
                st.batch_sizes.append(len(live))
                st.step_times.append(time.perf_counter())
                still = []
                for i, tok in zip(live, tokens):
                    out[i].append(int(tok))
                    st.new_tokens += 1
                    if finished(int(tok), len(out[i]), len(prompts[i]), params, self.max_positions):
                        self.stepper.free_slot(slot.pop(i))
                    else:
                        still.append(i)
                live = still
                if not live:
                    break
                logits = self.stepper.step([StepEntry(slot[i], [out[i][-1]], [0]) for i in live])
                tokens = self.picker(logits, live, [len(out[i]) for i in live], params)
            st.decode_seconds += time.perf_counter() - t0
        finally:
            for s in slot.values():          # only after an error: normal ends freed their slots above
                self.stepper.free_slot(s)

    def _ends_whatever_comes(self, n_new: int, prompt_len: int, params: GenParams) -> bool:
        """True when the request's token number `n_new` is its last one whatever its value is."""
        return n_new >= params.max_new_tokens or prompt_len + n_new >= self.max_positions

    def _run_batch_ahead(self, batch: list[int], prompts, params: GenParams, out: list[list[int]]) -> None:
        """The same batch with every decode step launched before the tokens of the step before it have
        been read on the host."""
        st = self.stats
        st.batches += 1
        slot = {}
        try:
            for i in batch:
                slot[i] = self.stepper.alloc_slot()
            t0 = time.perf_counter()
            live = list(batch)
            logits = self.stepper.step([StepEntry(slot[i], list(prompts[i]), [len(prompts[i]) - 1]) for i in live])
            picked = self.device_picker(logits, live, [0] * len(live), params)
            picked.start_copy()
            st.prompt_tokens += sum(len(prompts[i]) for i in live)
            first = True
            while True:
                # `picked` holds token number len(out[i]) + 1 of every request in `live`, still unread.
                # Launch the next step for the requests that this token cannot be the last of for a reason
                # known already (length); a stop token among them shows only when the tokens are read.
                ahead = [i for i in live if not self._ends_whatever_comes(len(out[i]) + 1, len(prompts[i]), params)]
                nxt = None
                if ahead:
                    rows = [live.index(i) for i in ahead] if len(ahead) != len(live) else None
                    toks_dev = picked.tokens if rows is None else picked.select(rows)
                    logits = self.stepper.step_decode_device([slot[i] for i in ahead], toks_dev)
                    nxt = self.device_picker(logits, ahead, [len(out[i]) + 1 for i in ahead], params)
                    nxt.start_copy()
                tokens = picked.to_host()                 # waits for the step before the one just launched
                if first:
                    st.prefill_seconds += time.perf_counter() - t0
                    t0, first = time.perf_counter(), False
                st.steps += 1
                st.batch_sizes.append(len(live))
                st.step_times.append(time.perf_counter())
                still = []
                for i, tok in zip(live, tokens):
                    out[i].append(int(tok))
                    st.new_tokens += 1
                    if finished(int(tok), len(out[i]), len(prompts[i]), params, self.max_positions):
                        self.stepper.free_slot(slot.pop(i))     # frees what the step ahead wrote for it, too
                    else:
                        still.append(i)
                if not still:
                    break
                if still != ahead:                        # somebody met a stop token: drop its row of the step ahead
                    keep = [ahead.index(i) for i in still]
                    nxt = nxt.narrowed(keep)
                live, picked = still, nxt
            st.decode_seconds += time.perf_counter() - t0
        finally:
            for s in slot.values():
                self.stepper.free_slot(s)
