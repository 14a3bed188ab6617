"""The generation loop's decisions with a scripted backend (no GPU): batching, stop tokens,
sequences that end earlier, slot hand-back, token accounting, capacity policy."""
import pytest

from cpp_minilamma_b200.engine.generate import Backend, GenerationError, generate, plan_batches


class Scripted(Backend):
    """Samples token = script[request][index]; records every step."""

    def __init__(self, scripts, n_slots=4, n_pages=100, max_positions=1000):
        self.scripts, self.n_slots, self.n_pages, self.max_positions = scripts, n_slots, n_pages, max_positions
        self.free = list(range(n_slots))
        self.held = set()
        self.log = []
        self.fed = {}

    def acquire(self, count):
        assert count <= len(self.free)
        slots = [self.free.pop(0) for _ in range(count)]
        self.held |= set(slots)
        for s in slots:
            self.fed[s] = []
        return slots

    def release(self, slot):
        assert slot in self.held, "released twice"
        self.held.discard(slot)
        self.free.append(slot)

    def step_and_sample(self, entries, requests, steps):
        assert len(entries) == len(requests) == len(steps)
        assert all(e.slot in self.held for e in entries)
        self.log.append([(r, list(e.tokens), list(e.want), s) for e, r, s in zip(entries, requests, steps)])
        for e in entries:
            self.fed[e.slot] += list(e.tokens)
        return [self.scripts[r][s] for r, s in zip(requests, steps)]


def test_prompts_in_one_step_then_one_token_each():
    scripts = {0: [10, 11, 12], 1: [20, 21, 22], 2: [30, 31, 32]}
    backend = Scripted(scripts)
    prompts = [[1, 2, 3, 4, 5], [6] * 9, [7, 8]]
    out = generate(backend, prompts, 3)
    assert [c.tokens for c in out] == [[10, 11, 12], [20, 21, 22], [30, 31, 32]]
    assert all(c.finish_reason == "length" for c in out)
    first = backend.log[0]
    assert [(r, t, w) for r, t, w, _ in first] == [(0, prompts[0], [4]), (1, prompts[1], [8]), (2, prompts[2], [1])]
    # 3 tokens cost the prompt step plus 2 decode steps; the last token is not fed back
    assert len(backend.log) == 3
    assert backend.log[1] == [(0, [10], [0], 1), (1, [20], [0], 1), (2, [30], [0], 1)]
    assert backend.log[2] == [(0, [11], [0], 2), (1, [21], [0], 2), (2, [31], [0], 2)]
    assert not backend.held


def test_stop_token_ends_a_sequence_early_and_is_not_emitted():
    scripts = {0: [10, 99, 12, 13], 1: [20, 21, 22, 23], 2: [99, 0, 0, 0]}
    backend = Scripted(scripts)
    out = generate(backend, [[1], [2, 3], [4]], 4, stop_ids={99})
    assert [c.tokens for c in out] == [[10], [20, 21, 22, 23], []]
    assert [c.finish_reason for c in out] == ["stop", "length", "stop"]
    assert [len(step) for step in backend.log] == [3, 2, 1, 1]   # the batch shrinks
    assert [r for r, *_ in backend.log[1]] == [0, 1]
    assert not backend.held
    again = Scripted(scripts)
    out = generate(again, [[1], [2, 3], [4]], 4, stop_ids={99}, ignore_eos=True)
    assert [c.tokens for c in out] == [[10, 99, 12, 13], [20, 21, 22, 23], [99, 0, 0, 0]]


def test_unequal_budgets_and_zero():
    scripts = {i: list(range(100 * i, 100 * i + 10)) for i in range(3)}
    backend = Scripted(scripts)
    out = generate(backend, [[1], [2], [3]], [1, 0, 4])
    assert [c.tokens for c in out] == [[0], [], [200, 201, 202, 203]]
    assert [c.finish_reason for c in out] == ["length"] * 3
    assert [r for r, *_ in backend.log[0]] == [0, 2]              # a request that wants nothing never runs
    assert len(backend.log) == 4


def test_more_requests_than_slots_run_in_batches_that_reuse_slots():
    scripts = {i: [i] * 3 for i in range(7)}
    backend = Scripted(scripts, n_slots=3)
    out = generate(backend, [[i + 1] for i in range(7)], 2)
    assert [c.tokens for c in out] == [[i, i] for i in range(7)]
    starts = [step for step in backend.log if step[0][3] == 0]
    assert [[r for r, *_ in step] for step in starts] == [[0, 1, 2], [3, 4, 5], [6]]
    assert not backend.held and sorted(backend.free) == [0, 1, 2]


def test_page_budget_limits_a_batch():
    assert plan_batches([64, 64, 64], [1, 1, 1], n_slots=8, n_pages=2) == [[0, 1], [2]]
    assert plan_batches([60, 60], [6, 5], n_slots=8, n_pages=2) == [[0], [1]]   # 65 held tokens: 2 pages; 64: 1
    assert plan_batches([60, 60], [6, 5], n_slots=8, n_pages=3) == [[0, 1]]
    assert plan_batches([1] * 5, [1] * 5, n_slots=8, n_pages=100, max_batch=2) == [[0, 1], [2, 3], [4]]
    with pytest.raises(GenerationError, match="pages"):
        plan_batches([200], [1], n_slots=8, n_pages=2)


def test_capacity_policy():
    backend = Scripted({0: [1] * 50}, max_positions=20)
    with pytest.raises(GenerationError, match="exceeds"):
        generate(backend, [[0] * 15], 10)
    out = generate(backend, [[0] * 15], 10, clip=True)
    assert len(out[0].tokens) == 5
    with pytest.raises(GenerationError, match="empty"):
        generate(backend, [[]], 1)
    with pytest.raises(GenerationError, match="one per prompt"):
        generate(backend, [[1]], [1, 2])


def test_slots_go_back_when_the_backend_fails():
    class Failing(Scripted):
        def step_and_sample(self, entries, requests, steps):
            if len(self.log) == 1:
                raise RuntimeError("boom")
            return super().step_and_sample(entries, requests, steps)

    backend = Failing({0: [1, 2, 3], 1: [4, 5, 6]})
    with pytest.raises(RuntimeError, match="boom"):
        generate(backend, [[1], [2]], 3)
    assert not backend.held


class ScriptedAhead(Scripted):
    """The same script behind `submit` / `submit_ahead` / `collect`: a step ahead takes its input
    tokens from what the previous step sampled ("on the device"), so it can be enqueued before
    the host has collected them.  Checks the contract of `submit_ahead`."""

    def __init__(self, *args, **kw):
        super().__init__(*args, **kw)
        self.pending = []          # tickets not yet collected
        self.last_step = None      # (slots, sampled tokens) of the latest submitted step
        self.ahead_calls = 0

    def submit(self, entries, requests, steps):
        sampled = Scripted.step_and_sample(self, entries, requests, steps)
        self.last_step = ([e.slot for e in entries], sampled)
        self.pending.append(sampled)
        assert len(self.pending) <= 2, "more than two steps in flight"
        return len(self.log) - 1

    def submit_ahead(self, slots, requests, steps):
        from cpp_minilamma_b200 import StepEntry
        assert self.last_step is not None and set(slots) <= set(self.last_step[0]), "a slot the previous step did not have"
        assert len(self.pending) == 1, "a step ahead goes out while exactly one step is uncollected"
        self.ahead_calls += 1
        sampled = dict(zip(*self.last_step))  # "on the device": by slot, whatever the order
        return self.submit([StepEntry(s, [sampled[s]], [0]) for s in slots], requests, steps)

    def collect(self, ticket):
        return self.pending.pop(0)

    def step_and_sample(self, entries, requests, steps):
        return self.collect(self.submit(entries, requests, steps))


@pytest.mark.parametrize("case", [
    dict(scripts={0: [10, 11, 12], 1: [20, 21, 22], 2: [30, 31, 32]}, prompts=[[1, 2, 3], [6] * 9, [7, 8]], budget=3, stops=()),
    dict(scripts={0: [10, 99, 12, 13], 1: [20, 21, 22, 23], 2: [99, 0, 0, 0]}, prompts=[[1], [2, 3], [4]], budget=4, stops=(99,)),
    dict(scripts={i: list(range(100 * i, 100 * i + 10)) for i in range(3)}, prompts=[[1], [2], [3]], budget=[1, 0, 4], stops=()),
    dict(scripts={0: [5, 6, 7, 8, 9, 99, 1], 1: [5, 99, 7, 8, 9, 10, 11], 2: [1, 2, 3, 4, 5, 6, 99]}, prompts=[[1], [2], [3]],
         budget=[7, 7, 6], stops=(99,)),
    dict(scripts={i: [i + 1] * 12 for i in range(6)}, prompts=[[1]] * 6, budget=[12, 3, 5, 1, 12, 2], stops=()),
])
def test_running_one_step_ahead_changes_no_result(case):
    plain, ahead = Scripted(case["scripts"]), ScriptedAhead(case["scripts"])
    a = generate(plain, case["prompts"], case["budget"], stop_ids=set(case["stops"]))
    b = generate(ahead, case["prompts"], case["budget"], stop_ids=set(case["stops"]))
    assert [(c.tokens, c.finish_reason) for c in a] == [(c.tokens, c.finish_reason) for c in b]
    assert not ahead.held and not ahead.pending
    # every token that a sequence was fed is one it kept (no row of an ended sequence leaks into a live one)
    kept = {r: list(case["prompts"][r]) + c.tokens for r, c in enumerate(b)}
    for step in ahead.log:
        for r, tokens, _, s in step:
            if s > 0:
                assert tokens == [case["scripts"][r][s - 1]]
    # a sequence that ends by length is in no step after its last: it is fed one token fewer than it keeps
    budgets = [case["budget"]] * len(case["prompts"]) if isinstance(case["budget"], int) else case["budget"]
    for r, completion in enumerate(b):
        if completion.finish_reason == "length" and budgets[r] > 0:
            fed = sum(1 for step in ahead.log for rr, _, _, s in step if rr == r and s > 0)
            assert fed == budgets[r] - 1, (r, fed)
    assert ahead.ahead_calls > 0 or all(n <= 2 for n in budgets)


def test_step_ahead_leaves_out_the_sequences_that_end_by_length():
    """Which sequences end by length with a step is known before its tokens are: the step ahead goes out without
    them, so a batch whose requests have different budgets stays one step ahead all the way."""
    scripts = {0: [10, 11, 12, 13, 14, 15], 1: [20, 21, 22, 23, 24, 25], 2: [30, 31, 32, 33, 34, 35]}
    backend = ScriptedAhead(scripts)
    out = generate(backend, [[1], [2, 2], [3]], [6, 3, 4])
    assert [c.tokens for c in out] == [scripts[0], scripts[1][:3], scripts[2][:4]]
    assert all(c.finish_reason == "length" for c in out)
    sizes = [len(step) for step in backend.log]
    assert sizes == [3, 3, 3, 2, 1, 1]           # the prompt step, then the batch as it shrinks
    assert backend.ahead_calls == 5               # every decode step went out ahead of the host
    assert not backend.held and not backend.pending


def test_step_ahead_rows_of_a_stopped_sequence_are_dropped():
    scripts = {0: [10, 99, 12, 13, 14], 1: [20, 21, 22, 23, 24]}
    backend = ScriptedAhead(scripts)
    out = generate(backend, [[1], [2]], 5, stop_ids={99})
    assert [c.tokens for c in out] == [[10], [20, 21, 22, 23, 24]]
    # request 0 stopped at its second token; the step that was already ahead fed it once more (dropped)
    fed_to_0 = [tokens for step in backend.log for r, tokens, _, _ in step if r == 0]
    assert fed_to_0 == [[1], [10], [99]]
    fed_to_1 = [tokens for step in backend.log for r, tokens, _, _ in step if r == 1]
    assert fed_to_1 == [[2], [20], [21], [22], [23]]
    # the stop cost no step sent from the host's side of the tokens: only the prompt step was not a step ahead
    assert len(backend.log) - backend.ahead_calls == 1


@pytest.mark.parametrize("backend_kind", [Scripted, ScriptedAhead])
def test_statistics_count_steps_and_stamp_each_step(backend_kind):
    """`stats` counts the prompt step and the decode steps and carries one host time per step whose tokens
    reached the host (the prompt step first): what the bench reads its end-to-end figure from."""
    scripts = {0: [10, 11, 12, 13, 14, 15], 1: [20, 21, 22, 23, 24, 25]}
    backend = backend_kind(scripts)
    stats = {}
    out = generate(backend, [[1, 2, 3], [4]], 6, stats=stats)
    assert [c.tokens for c in out] == [scripts[0], scripts[1]]
    assert stats["prefill_steps"] == 1 and stats["prefill_tokens"] == 4
    assert stats["decode_steps"] == 5 and stats["decode_tokens"] == 10
    stamps = stats["step_stamps"]
    assert len(stamps) == 6 and all(b >= a for a, b in zip(stamps, stamps[1:]))
    assert stats["decode_s"] >= stamps[-1] - stamps[0] >= 0.0
