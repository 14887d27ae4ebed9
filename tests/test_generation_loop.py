"""The generation loop's decisions, with a device that is not there: which steps are
launched for whom, when sequences end, how a queue is cut into batches, what is given back."""

import pytest

from thing_htn_2026_b200.engine.generation import (Completion, GenerationLoop, Request, form_batches,
                                                   tokens_needed)


class FakeBackend:
    """Sequence i's n-th token is 100 * (i + 1) + n, or what ``script`` says.  Records every
    call."""

    page_size = 64

    def __init__(self, capacity_tokens=4096, max_batch=8, script=None):
        self._capacity, self._max_batch = capacity_tokens, max_batch
        self.script = script or {}
        self.calls = []
        self.open_slots = set()
        self.next_slot = 0
        self.count = {}
        self.fetched = 0

    def capacity_tokens(self):
        return self._capacity

    def max_batch(self):
        return self._max_batch

    def open_batch(self, requests):
        slots = list(range(self.next_slot, self.next_slot + len(requests)))
        self.next_slot += len(requests)
        assert not self.open_slots, "a batch was opened before the last one was closed"
        self.open_slots.update(slots)
        self.first = slots[0]
        self.count = {s: 0 for s in slots}
        self.calls.append(("open", len(requests)))
        return slots

    def _tokens(self, slots):
        out = []
        for s in slots:
            i, n = s - self.first, self.count[s]
            out.append(self.script.get((i, n), 100 * (i + 1) + n))
            self.count[s] += 1
        return out

    def launch_prefill(self, slots, prompts):
        self.calls.append(("prefill", tuple(s - self.first for s in slots), tuple(len(p) for p in prompts)))
        return self._tokens(slots)

    def launch_decode(self, slots):
        assert set(slots) <= self.open_slots
        self.calls.append(("decode", tuple(s - self.first for s in slots)))
        return self._tokens(slots)

    def fetch(self, handle):
        self.fetched += 1
        return handle

    def close_batch(self, slots):
        assert set(slots) == self.open_slots
        self.open_slots.clear()
        self.calls.append(("close", len(slots)))

    def decodes(self):
        return [c[1] for c in self.calls if c[0] == "decode"]


def run(backend, requests, depth=3):
    loop = GenerationLoop(backend, depth)
    steps = list(loop.run_batch(requests))
    return loop, steps


def test_fixed_count_yields_exactly_n_steps_and_n_minus_1_decodes():
    backend = FakeBackend()
    loop, steps = run(backend, [Request([1, 2, 3], 6), Request([4], 6)])
    assert len(steps) == 6 and all(len(s) == 2 and all(type(t) is int for t in s) for s in steps)
    assert [s[0] for s in steps] == [100, 101, 102, 103, 104, 105]
    assert loop.decode_launches == 5 and backend.decodes() == [(0, 1)] * 5
    assert backend.calls[0] == ("open", 2) and backend.calls[1] == ("prefill", (0, 1), (3, 1))
    assert backend.calls[-1] == ("close", 2)


@pytest.mark.parametrize("depth", [1, 2, 3, 5])
def test_never_launches_a_step_that_cannot_be_needed(depth):
    backend = FakeBackend()
    loop, steps = run(backend, [Request([1], 4), Request([2], 1), Request([3], 7)], depth)
    assert loop.decode_launches == 6                               # longest limit - 1
    assert backend.decodes() == [(0, 2)] * 3 + [(2,)] * 3          # shorter ones leave when their limit is reached
    assert [len([t for t in col if t is not None]) for col in zip(*steps)] == [4, 1, 7]
    assert steps[0] == [100, 200, 300] and steps[1] == [101, None, 301] and steps[-1] == [None, None, 306]


def test_stop_token_ends_a_sequence_and_the_rest_goes_on():
    backend = FakeBackend(script={(0, 2): 7})
    completions = [Completion(), Completion()]
    loop = GenerationLoop(backend, depth=1)
    steps = list(loop.run_batch([Request([1], 10, stop_token_ids=(7,)), Request([2], 5)], completions))
    assert completions[0].tokens == [100, 101, 7] and completions[0].finish_reason == "stop"
    assert completions[1].tokens == [200, 201, 202, 203, 204] and completions[1].finish_reason == "length"
    assert len(steps) == 5 and steps[3] == [None, 203]
    # with one step in flight ahead of the host, sequence 0 rides along for one step after its stop
    assert backend.decodes() == [(0, 1), (0, 1), (0, 1), (1,)]


def test_tokens_launched_before_a_stop_was_seen_are_dropped():
    backend = FakeBackend(script={(0, 1): 7})
    completions = [Completion()]
    list(GenerationLoop(backend, depth=4).run_batch([Request([1], 50, stop_token_ids=(7,))], completions))
    assert completions[0].tokens == [100, 7]
    assert len(backend.decodes()) <= 1 + 4 + 1 and backend.fetched == len(backend.decodes()) + 1
    assert backend.calls[-1] == ("close", 1)


def test_zero_limit_and_empty_batch():
    backend = FakeBackend()
    assert list(GenerationLoop(backend).run_batch([])) == []
    assert list(GenerationLoop(backend).run_batch([Request([1], 0)])) == []
    assert backend.calls == []
    loop, steps = run(backend, [Request([1], 0), Request([2], 2)])
    assert steps == [[None, 200], [None, 201]]
    assert backend.calls[1] == ("prefill", (1,), (1,))


def test_slots_are_given_back_when_the_consumer_stops_early():
    backend = FakeBackend()
    generator = GenerationLoop(backend).run_batch([Request([1], 100)])
    next(generator)
    generator.close()
    assert backend.calls[-1] == ("close", 1) and not backend.open_slots


def test_request_validation():
    with pytest.raises(ValueError, match="prompt token"):
        Request([], 3)
    with pytest.raises(ValueError, match="max_new_tokens"):
        Request([1], -1)
    with pytest.raises(ValueError, match="temperature"):
        Request([1], 1, temperature=-0.5)


def test_queue_is_cut_into_batches_that_fit():
    assert tokens_needed(Request([0] * 60, 5), 64) == 64 and tokens_needed(Request([0] * 60, 6), 64) == 128
    requests = [Request([0] * n, 10) for n in (10, 100, 30, 500, 20, 20, 20)]
    assert form_batches(requests, capacity_tokens=640, max_batch=3, page_size=64) == [[0, 1, 2], [3, 4, 5], [6]]
    assert form_batches(requests, capacity_tokens=600, max_batch=3, page_size=64) == [[0, 1, 2], [3, 4], [5, 6]]
    assert form_batches(requests, capacity_tokens=10 ** 6, max_batch=100, page_size=64) == [[0, 1, 2, 3, 4, 5, 6]]
    with pytest.raises(ValueError, match="request 3 needs"):
        form_batches(requests, capacity_tokens=256, max_batch=3, page_size=64)


def test_generate_all_runs_batches_one_after_another():
    backend = FakeBackend(capacity_tokens=192, max_batch=2)
    requests = [Request([0] * 5, 3), Request([0] * 70, 2), Request([0] * 5, 4), Request([0] * 5, 1), Request([0], 2)]
    loop = GenerationLoop(backend, depth=2)
    done = loop.generate_all(requests)
    assert loop.batches_run == [[0, 1], [2, 3], [4]]
    assert [len(c.tokens) for c in done] == [3, 2, 4, 1, 2] and all(c.finish_reason == "length" for c in done)
    kinds = [c[0] for c in backend.calls if c[0] in ("open", "close")]
    assert kinds == ["open", "close"] * 3                    # a batch ends before the next one starts


@pytest.mark.parametrize("depth", [1, 3, 9])
def test_never_more_than_depth_plus_one_unfetched_steps(depth):
    """The device backend's ring of pinned token buffers is sized from this bound."""
    class Counting(FakeBackend):
        outstanding = worst = 0

        def launch_prefill(self, slots, prompts):
            self.outstanding += 1
            self.worst = max(self.worst, self.outstanding)
            return super().launch_prefill(slots, prompts)

        def launch_decode(self, slots):
            self.outstanding += 1
            self.worst = max(self.worst, self.outstanding)
            return super().launch_decode(slots)

        def fetch(self, handle):
            self.outstanding -= 1
            return super().fetch(handle)

    backend = Counting()
    run(backend, [Request([1, 2, 3], 40), Request([4], 25)], depth=depth)
    assert backend.outstanding == 0 and backend.worst == depth + 1
