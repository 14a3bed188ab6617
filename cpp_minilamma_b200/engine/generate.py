"""The generation loop: batches of unequal prompts, stop tokens, sequences that end early.

Shape of the loop, per batch (the reference runs it for one sequence,
app/backend_cli.cc:161-176): all prompts in one step, sample one token per sequence from
the logits of its last prompt token, then one step per further token with one token per
live sequence.  N generated tokens cost N - 1 decode steps: the last sampled token is
not fed back (app/backend_cli.cc:172).  A sampled stop token ends its sequence and is not
emitted (app/backend_cli.cc:170); the sequence then leaves the batch and its slot goes
back to the cache, while the others go on.  Requests that do not fit into one batch run
in further batches, which reuse the slots.

The loop talks to a small backend interface (`acquire`, `release`, `step_and_sample`,
limits), so its decisions can be tested without a device.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Set

from ..cache.paged import PAGE
from .step import StepEntry


class GenerationError(ValueError):
    pass


@dataclass
class Completion:
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""  # "stop" (a stop token was sampled) or "length"


class Backend:
    """What the loop needs from an engine."""

    n_slots: int        # sequences that can be live together
    n_pages: int        # pages of PAGE tokens that live sequences can hold together
    max_positions: int  # longest sequence the model can hold

    def acquire(self, count: int) -> List[int]:
        raise NotImplementedError

    def release(self, slot: int) -> None:
        raise NotImplementedError

    def step_and_sample(self, entries: Sequence[StepEntry], requests: Sequence[int],
                        steps: Sequence[int]) -> List[int]:
        """Run the step; sample one token per entry from the logits at its wanted place."""
        raise NotImplementedError


def plan_batches(prompt_lens: Sequence[int], max_new: Sequence[int], n_slots: int, n_pages: int,
                 max_batch: Optional[int] = None) -> List[List[int]]:
    """Cut the requests, in order, into batches that fit the slots and the page budget.

    A request needs pages for its prompt plus all tokens it may generate but one (the
    last sampled token is never fed back)."""
    limit = n_slots if max_batch is None else min(n_slots, max_batch)
    if limit < 1:
        raise GenerationError("no slot to run a request in")
    batches: List[List[int]] = []
    current: List[int] = []
    used = 0
    for i, (p, n) in enumerate(zip(prompt_lens, max_new)):
        held = p + max(n - 1, 0)
        pages = (held + PAGE - 1) // PAGE
        if pages > n_pages:
            raise GenerationError(
                f"request {i}: {held} tokens need {pages} pages, the cache has {n_pages}")
        if current and (len(current) == limit or used + pages > n_pages):
            batches.append(current)
            current, used = [], 0
        current.append(i)
        used += pages
    if current:
        batches.append(current)
    return batches


def generate(backend: Backend, prompts: Sequence[Sequence[int]], max_new_tokens, stop_ids: Set[int] = frozenset(),
             ignore_eos: bool = False, max_batch: Optional[int] = None, clip: bool = False,
             stats: Optional[dict] = None) -> List[Completion]:
    """Generate for every prompt; results come back in request order.

    max_new_tokens: one number for all requests or one per request.  A request whose
    prompt plus new tokens exceeds the model's positions is an error (the reference's
    "prompt + n-predict exceeds context window", app/backend_cli.cc:146-148) unless
    `clip` shortens it (its legacy bench clips, app/main.cc:170).  `stats`, when given,
    receives wall-clock seconds and counts of the prompt steps and of the decode steps
    (sampling included, as the caller sees them), and `step_stamps`, the host time at which
    each step's tokens arrived (the prompt step's first).
    """
    n_requests = len(prompts)
    if isinstance(max_new_tokens, int):
        budgets = [max_new_tokens] * n_requests
    else:
        budgets = list(max_new_tokens)
        if len(budgets) != n_requests:
            raise GenerationError("max_new_tokens must be one number or one per prompt")
    for i, (prompt, n) in enumerate(zip(prompts, budgets)):
        if len(prompt) < 1:
            raise GenerationError(f"request {i}: the prompt is empty")
        if n < 0:
            raise GenerationError(f"request {i}: max_new_tokens must be >= 0")
        if len(prompt) > backend.max_positions:
            raise GenerationError(f"request {i}: the prompt of {len(prompt)} tokens exceeds the "
                                  f"{backend.max_positions} positions of the model")
        if len(prompt) + n > backend.max_positions:
            if not clip:
                raise GenerationError(f"request {i}: prompt ({len(prompt)}) + max_new_tokens ({n}) exceeds the "
                                      f"{backend.max_positions} positions of the model")
            budgets[i] = backend.max_positions - len(prompt)
    stops = set() if ignore_eos else set(stop_ids)
    results = [Completion() for _ in range(n_requests)]
    active = [i for i in range(n_requests) if budgets[i] > 0]
    for i in range(n_requests):
        if budgets[i] == 0:
            results[i].finish_reason = "length"
    batches = plan_batches([len(prompts[i]) for i in active], [budgets[i] for i in active],
                           backend.n_slots, backend.n_pages, max_batch)
    for batch in batches:
        requests = [active[j] for j in batch]
        _run_batch(backend, requests, prompts, budgets, stops, results, stats)
    return results


def _run_batch(backend, requests, prompts, budgets, stops, results, stats=None) -> None:
    """One batch from its prompts to its last token.

    A backend that has `submit`, `submit_ahead` and `collect` is kept one step ahead: while
    the host looks at the tokens of step t, step t + 1 (fed on the device with those same
    tokens) is already running.  The step ahead holds the sequences that cannot end by length
    at step t (those that do are known beforehand and left out).  If one of them ends by a
    stop token at step t, the step ahead has a row for it all the same; that row is dropped when
    the step is collected, and the step after it goes out without the sequence - the device never
    waits for the host."""
    slots = backend.acquire(len(requests))
    live = dict(zip(requests, slots))  # request -> slot, in request order
    submit = getattr(backend, "submit", None)
    ahead = getattr(backend, "submit_ahead", None) if submit is not None else None
    last = {}

    def apply(rows, sampled):
        """Take one sampled token per request of `rows` that is still live (a row of a sequence that has
        ended since the step was sent is dropped); returns the requests that go on."""
        goes_on = []
        for r, token in zip(rows, sampled):
            if r not in live:
                continue
            done = None
            if token in stops:
                done = "stop"
            else:
                results[r].tokens.append(int(token))
                if len(results[r].tokens) >= budgets[r]:
                    done = "length"
            if done:
                results[r].finish_reason = done
                backend.release(live.pop(r))
            else:
                last[r] = int(token)
                goes_on.append(r)
        return goes_on

    def count(kind, n_tokens):
        if stats is not None:
            stats[kind + "_steps"] = stats.get(kind + "_steps", 0) + 1
            stats[kind + "_tokens"] = stats.get(kind + "_tokens", 0) + n_tokens

    try:
        rows = list(live)  # the requests of the step in flight, in the order of its rows
        entries = [StepEntry(live[r], list(prompts[r]), [len(prompts[r]) - 1]) for r in rows]
        began = time.perf_counter()
        step = 0
        count("prefill", sum(len(e.tokens) for e in entries))
        ticket = submit(entries, rows, [0] * len(rows)) if submit else None
        decode_began = None
        while True:
            spec, spec_rows = None, None
            if ahead is not None:
                # who goes on whatever this step samples, unless it is a stop token: the others end with this step
                spec_rows = [r for r in rows if r in live and len(results[r].tokens) + 1 < budgets[r]]
                if spec_rows:
                    spec = ahead([live[r] for r in spec_rows], spec_rows, [step + 1] * len(spec_rows))
                    if spec is not None:
                        count("decode", len(spec_rows))
            sampled = backend.collect(ticket) if submit else backend.step_and_sample(entries, rows, [step] * len(rows))
            if decode_began is None:
                decode_began = time.perf_counter()
                if stats is not None:
                    stats["prefill_s"] = stats.get("prefill_s", 0.0) + decode_began - began
            if stats is not None:  # when each step's tokens reached the host: the prompt step first
                stats.setdefault("step_stamps", []).append(time.perf_counter())
            goes_on = apply(rows, sampled)
            step += 1
            if spec is not None:  # the step ahead is the next step; rows of sequences that just stopped are dropped then
                ticket, rows = spec, spec_rows
                continue
            if not goes_on:
                break
            rows = goes_on
            entries = [StepEntry(live[r], [last[r]], [0]) for r in rows]
            count("decode", len(rows))
            if submit:
                ticket = submit(entries, rows, [step] * len(rows))
        if stats is not None and decode_began is not None:
            # everything after the prompt step: decode steps, sampling, host bookkeeping
            stats["decode_s"] = stats.get("decode_s", 0.0) + time.perf_counter() - decode_began
    finally:
        for slot in live.values():
            backend.release(slot)
