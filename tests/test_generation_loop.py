"""The generation loop's decisions (CPU), with a scripted backend in place of
the engine: batching, stop tokens, sequences that end earlier, slots given
back, one batch after another."""
import pytest

from mivi_v4_b200.engine import GenerationError, plan_batches, run_generation
from mivi_v4_b200.engine.generate import Request


class Scripted:
    """Emits for request i the tokens of script[i], one per call."""

    def __init__(self, script, max_batch=4, total_pages=64, page_size=4, max_positions=None):
        self.script, self.max_batch, self.total_pages = script, max_batch, total_pages
        self.page_size, self.max_positions = page_size, max_positions
        self.open_handles, self.next_handle, self.calls, self.peak = set(), 0, [], 0
        self.lengths = {}

    def open(self):
        assert len(self.open_handles) < self.max_batch, "more sequences than slots"
        h = self.next_handle
        self.next_handle += 1
        self.open_handles.add(h)
        self.lengths[h] = 0
        return h

    def close(self, h):
        assert h in self.open_handles, "closed twice"
        self.open_handles.remove(h)

    def forward_and_sample(self, requests, token_lists):
        assert all(r.handle in self.open_handles for r in requests)
        self.calls.append([(r.index, list(t)) for r, t in zip(requests, token_lists)])
        for r, t in zip(requests, token_lists):
            self.lengths[r.handle] += len(t)
        self.peak = max(self.peak, len(self.open_handles))
        return [self.script[r.index][len(r.output)] for r in requests]


def test_prompts_in_one_step_then_one_token_each():
    b = Scripted({0: [5, 6, 7, 8], 1: [9, 9, 9, 9]})
    out = run_generation([[1, 2, 3], [4]], 3, b)
    assert [r.output for r in out] == [[5, 6, 7], [9, 9, 9]]
    assert b.calls[0] == [(0, [1, 2, 3]), (1, [4])]
    assert b.calls[1] == [(0, [5]), (1, [9])]
    assert len(b.calls) == 3                      # no forward pass after the last sampled token
    assert not b.open_handles
    assert [r.finish_reason for r in out] == ["length", "length"]


def test_stop_token_is_not_emitted_and_ends_only_its_sequence():
    b = Scripted({0: [5, 99, 7, 8], 1: [6, 6, 6, 99], 2: [99]})
    out = run_generation([[1], [2], [3]], 4, b, stop_ids=[99])
    assert [r.output for r in out] == [[5], [6, 6, 6], []]
    assert [r.finish_reason for r in out] == ["stop", "stop", "stop"]
    assert [[i for i, _ in c] for c in b.calls] == [[0, 1, 2], [0, 1], [1], [1]]
    assert not b.open_handles


def test_batches_one_after_another_reuse_slots():
    script = {i: [10 + i] * 8 for i in range(5)}
    b = Scripted(script, max_batch=2)
    out = run_generation([[1]] * 5, [1, 3, 2, 2, 1], b)
    assert [len(r.output) for r in out] == [1, 3, 2, 2, 1]
    assert b.peak <= 2 and not b.open_handles
    firsts = [c for c in b.calls if any(t == [1] for _, t in c)]
    assert [[i for i, _ in c] for c in firsts] == [[0, 1], [2, 3], [4]]


def test_batches_fit_the_cache():
    reqs = [Request(i, [0] * n, m) for i, (n, m) in enumerate([(10, 6), (3, 1), (8, 8), (1, 3)])]
    assert [[r.index for r in b] for b in plan_batches(reqs, 8, 6, 4)] == [[0, 1], [2, 3]]
    with pytest.raises(GenerationError, match="need 7 pages"):
        plan_batches([Request(0, [0] * 20, 8)], 8, 6, 4)


def test_zero_new_tokens_and_empty_prompt():
    b = Scripted({0: [5], 1: [6]})
    out = run_generation([[1], [2]], [0, 1], b)
    assert [r.output for r in out] == [[], [6]]
    assert b.calls == [[(1, [2])]] or b.calls[0] == [(1, [2])]
    with pytest.raises(GenerationError, match="empty prompt"):
        run_generation([[]], 1, Scripted({0: [1]}))


def test_context_end_stops_sampling():
    b = Scripted({0: [5] * 10}, max_positions=5)
    out = run_generation([[1, 2, 3]], 10, b)
    # 3 prompt tokens; tokens sampled while the cache holds 3 and 4 tokens; at 5 it is full
    assert out[0].output == [5, 5] and out[0].finish_reason == "context"
    with pytest.raises(GenerationError, match="context"):
        run_generation([[1] * 6], 1, Scripted({0: [1]}, max_positions=5))


def test_slots_go_back_when_the_backend_fails():
    class Failing(Scripted):
        def forward_and_sample(self, requests, token_lists):
            if len(self.calls) == 1:
                raise RuntimeError("boom")
            return super().forward_and_sample(requests, token_lists)
    b = Failing({0: [1, 1], 1: [2, 2]})
    with pytest.raises(RuntimeError):
        run_generation([[1], [2]], 2, b)
    assert not b.open_handles
