"""The generation loop's decisions, with a scripted stepper in place of the GPU engine (CPU)."""
import pytest

from garlic_inference_b200.engine import (GenerationError, GenerationLoop, GenParams, finished, plan_batches,
                                          tokens_held)


class ScriptedStepper:
    """Stands in for the engine: 'logits' are the lists of (slot, fed tokens); the picker turns them
    into the next token by a rule of the test.  Records every call."""

    def __init__(self, n_slots=4):
        self.free = list(range(n_slots - 1, -1, -1))
        self.live = {}
        self.calls = []
        self.freed = []

    def alloc_slot(self):
        s = self.free.pop()
        self.live[s] = 0
        return s

    def free_slot(self, s):
        assert s in self.live, "slot freed twice or never given out"
        del self.live[s]
        self.free.append(s)
        self.freed.append(s)

    def step(self, entries):
        for e in entries:
            assert e.slot in self.live
            self.live[e.slot] += len(e.tokens)
        self.calls.append([(e.slot, list(e.tokens), list(e.want)) for e in entries])
        return [(e.slot, list(e.tokens)) for e in entries]


def counting_picker(log):
    """Next token = last fed token + 1; logs (request ids, token indices) it was keyed with."""
    def pick(logits, request_ids, token_indices, params):
        log.append((list(request_ids), list(token_indices)))
        return [toks[-1] + 1 for _, toks in logits]
    return pick


def loop(stepper, picker, capacity=4096, max_positions=1000, max_batch=4):
    return GenerationLoop(stepper, picker, capacity, max_positions, max_batch)


def test_unequal_prompts_one_prefill_then_one_token_each():
    st, log = ScriptedStepper(), []
    out = loop(st, counting_picker(log)).run([[10, 11, 12], [50], [70, 71]], GenParams(max_new_tokens=3))
    assert out == [[13, 14, 15], [51, 52, 53], [72, 73, 74]]
    assert st.calls[0] == [(0, [10, 11, 12], [2]), (1, [50], [0]), (2, [70, 71], [1])]
    assert st.calls[1] == [(0, [13], [0]), (1, [51], [0]), (2, [72], [0])]
    assert len(st.calls) == 3                      # the last token of each request is never fed back
    assert log == [([0, 1, 2], [0, 0, 0]), ([0, 1, 2], [1, 1, 1]), ([0, 1, 2], [2, 2, 2])]
    assert not st.live and sorted(st.freed) == [0, 1, 2]


def test_stop_token_ends_a_request_early_and_the_batch_shrinks():
    st = ScriptedStepper()
    lp = loop(st, counting_picker([]))
    out = lp.run([[1], [20], [97]], GenParams(max_new_tokens=6, stop_token_ids=(22, 98)))
    assert out == [[2, 3, 4, 5, 6, 7], [21, 22], [98]]          # the stop token is the last one returned
    assert [len(c) for c in st.calls] == [3, 2, 1, 1, 1, 1]
    assert st.freed == [2, 1, 0]                                # given back as each ends
    assert lp.stats.batch_sizes == [3, 2, 1, 1, 1, 1] and lp.stats.new_tokens == 9
    assert lp.stats.prompt_tokens == 3 and lp.stats.batches == 1


def test_more_requests_than_the_batch_holds_run_as_batches_one_after_another():
    st = ScriptedStepper(n_slots=2)
    lp = loop(st, counting_picker([]), max_batch=2)
    prompts = [[i * 10] for i in range(5)]
    out = lp.run(prompts, GenParams(max_new_tokens=2))
    assert out == [[i * 10 + 1, i * 10 + 2] for i in range(5)]
    assert lp.stats.batches == 3
    prefill_calls = [c for c in st.calls if c[0][2] == [0] and len(c[0][1]) == 1 and c[0][1][0] % 10 == 0]
    assert [len(c) for c in prefill_calls] == [2, 2, 1]
    assert set(s for c in st.calls for s, _, _ in c) == {0, 1}          # two slots, used again
    assert not st.live


def test_capacity_cuts_batches_and_refuses_what_never_fits():
    assert tokens_held(100, 30, 4096) == 192 and tokens_held(1, 1, 4096) == 64
    assert tokens_held(4000, 500, 4096) == 4096
    assert plan_batches([100, 100, 100], 29, 256, 4096, 8) == [[0, 1], [2]]
    assert plan_batches([10] * 5, 5, 4096, 4096, 2) == [[0, 1], [2, 3], [4]]
    with pytest.raises(GenerationError, match="request 1 may hold 320"):
        plan_batches([10, 300], 10, 256, 4096, 8)
    with pytest.raises(GenerationError, match="empty prompt"):
        plan_batches([3, 0], 10, 256, 4096, 8)
    with pytest.raises(GenerationError, match="takes 64 positions"):
        plan_batches([65], 1, 256, 64, 8)


def test_finish_rules():
    p = GenParams(max_new_tokens=4, stop_token_ids=[7])
    assert finished(7, 1, 10, p, 100) and finished(3, 4, 10, p, 100) and not finished(3, 3, 10, p, 100)
    assert finished(3, 2, 98, p, 100) and not finished(3, 1, 98, p, 100)     # positions run out
    with pytest.raises(GenerationError):
        GenParams(max_new_tokens=-1)
    with pytest.raises(GenerationError):
        GenParams(temperature=-0.5)


def test_positions_limit_ends_generation():
    st = ScriptedStepper()
    out = loop(st, counting_picker([]), max_positions=6).run([[1, 2, 3, 4]], GenParams(max_new_tokens=50))
    assert out == [[5, 6]] and st.live == {}
    assert max(sum(len(t) for s, t, _ in c) for c in st.calls) <= 4


def test_zero_new_tokens_and_no_prompts_touch_nothing():
    st = ScriptedStepper()
    assert loop(st, counting_picker([])).run([[1, 2]], GenParams(max_new_tokens=0)) == [[]]
    assert loop(st, counting_picker([])).run([], GenParams()) == []
    assert st.calls == []


def test_slots_are_given_back_when_a_step_fails():
    class Failing(ScriptedStepper):
        def step(self, entries):
            if len(self.calls) == 1:
                raise RuntimeError("boom")
            return super().step(entries)

    st = Failing()
    with pytest.raises(RuntimeError, match="boom"):
        loop(st, counting_picker([])).run([[1], [2]], GenParams(max_new_tokens=5))
    assert not st.live and len(st.free) == 4


# ---- the loop that runs one step ahead of the host --------------------------------------------
class AheadStepper(ScriptedStepper):
    """A stepper that also takes a step's tokens 'from the device' (here: a list nobody has read yet)."""

    def __init__(self, n_slots=4):
        super().__init__(n_slots)
        self.ahead_calls = []

    def step_decode_device(self, slots, tokens):
        for s in slots:
            assert s in self.live, "a step ahead for a slot that has been given back"
            self.live[s] += 1
        toks = list(tokens)
        assert len(toks) == len(slots)
        self.ahead_calls.append([(s, t) for s, t in zip(slots, toks)])
        return [(s, [t]) for s, t in zip(slots, toks)]


class FakePicked:
    def __init__(self, tokens, log):
        self.tokens, self.log, self.copied = list(tokens), log, False

    def start_copy(self):
        self.copied = True

    def to_host(self):
        assert self.copied, "tokens read before their copy was started"
        self.log.append(("read", list(self.tokens)))
        return list(self.tokens)

    def select(self, rows):
        return [self.tokens[r] for r in rows]

    def narrowed(self, rows):
        p = FakePicked([self.tokens[r] for r in rows], self.log)
        p.copied = True
        return p


def ahead_picker(log, keys):
    def pick(logits, request_ids, token_indices, params):
        keys.append((list(request_ids), list(token_indices)))
        return FakePicked([toks[-1] + 1 for _, toks in logits], log)
    return pick


@pytest.mark.parametrize("prompts,params", [
    ([[10, 11, 12], [50], [70, 71]], GenParams(max_new_tokens=3)),
    ([[1], [20], [97]], GenParams(max_new_tokens=6, stop_token_ids=(22, 98))),
    ([[1], [20], [97]], GenParams(max_new_tokens=1)),
    ([[5], [30]], GenParams(max_new_tokens=9, stop_token_ids=(8, 33, 34))),
])
def test_running_one_step_ahead_returns_what_the_plain_loop_returns(prompts, params):
    plain_st, plain_keys = ScriptedStepper(), []
    want = loop(plain_st, counting_picker(plain_keys)).run(prompts, params)
    st, log, keys = AheadStepper(), [], []
    lp = GenerationLoop(st, None, 4096, 1000, 4, device_picker=ahead_picker(log, keys))
    got = lp.run(prompts, params)
    assert got == want
    assert not st.live and sorted(st.freed) == sorted(plain_st.freed)
    assert lp.stats.new_tokens == sum(len(o) for o in want)
    # every token that was kept was drawn with the same (request, token index) key as in the plain loop
    kept = {(r, i) for ids, idx in plain_keys for r, i in zip(ids, idx)}
    drawn = {(r, i) for ids, idx in keys for r, i in zip(ids, idx)}
    assert kept <= drawn


def test_one_step_ahead_launches_before_it_reads_and_never_steps_past_a_known_end():
    st, log, keys = AheadStepper(), [], []
    lp = GenerationLoop(st, None, 4096, 1000, 4, device_picker=ahead_picker(log, keys))
    out = lp.run([[1], [20]], GenParams(max_new_tokens=3, stop_token_ids=(22,)))
    assert out == [[2, 3, 4], [21, 22]]
    # step for token 2 of both requests is launched before token 1 is read; request 1 meets its stop token at
    # token 2, which shows only after the step for token 3 has taken it along: that row is dropped
    assert st.ahead_calls == [[(0, 2), (1, 21)], [(0, 3), (1, 22)]]
    assert len(st.calls) == 1                     # the prompts' step; everything after it came from the device
    assert st.freed == [1, 0]


def test_one_step_ahead_respects_the_position_limit():
    st, log, keys = AheadStepper(), [], []
    lp = GenerationLoop(st, None, 4096, 5, 4, device_picker=ahead_picker(log, keys))
    out = lp.run([[1, 2, 3]], GenParams(max_new_tokens=10))
    assert out == [[4, 5]]                        # 3 + 2 = 5 positions
    assert st.live == {} and max(len(c) for c in st.ahead_calls) == 1 and len(st.ahead_calls) == 1


def test_timeline_finds_the_repeating_layer():
    """The timeline's reading of its marks: entries in launch order, and the period of the launch sizes."""
    import torch
    from garlic_inference_b200.engine import timeline
    head, layer, tail = [(1, 32)], [(8, 256), (384, 256), (96, 128), (256, 160)], [(148, 192), (8, 32)]
    assert timeline.period(head + layer * 12 + tail) == 4
    assert timeline.period([(i, 32) for i in range(40)]) == 0
    buf = torch.zeros(4 + 4 * timeline.ENTRIES, dtype=torch.int64)
    buf[0], buf[1] = 2, 2
    buf[4:8] = torch.tensor([1000, 1500, (3 << 16) | 128, 0])
    buf[8:12] = torch.tensor([2000, 4500, (7 << 16) | 64, 0])
    assert timeline.read(buf) == [(3, 128, 0.0, 0.5), (7, 64, 1.0, 3.5)]
