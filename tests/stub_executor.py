"""An executor without a model: the next token is a function of the last token and its
position, so any difference between scheduling orders is a scheduling fault. It uses the
real cache manager, and checks that what it is asked to run is consistent with it."""

from __future__ import annotations

from paged_attention_engine_b200.cache import CacheManager, KVGroupSpec
from paged_attention_engine_b200.engine.scheduler import WorkResult


def next_token(last: int, position: int) -> int:
    return (31 * last + 17 * position + 5) % 97


def expected_tokens(prompt, count: int) -> tuple[int, ...]:
    history = list(prompt)
    for _ in range(count):
        history.append(next_token(history[-1], len(history) - 1))
    return tuple(history[len(prompt):])


def make_manager(num_blocks: int, block_size: int, max_requests: int = 64, window: int = 0) -> CacheManager:
    groups = [KVGroupSpec(1, 8, 0, (0,))]
    if window:
        groups.append(KVGroupSpec(1, 8, window, (1,)))
    return CacheManager(groups, num_blocks, block_size, max_requests)


class _Later:
    """Tokens that the scheduler may only ask for after the step has been handed over."""

    def __init__(self, tokens):
        self._tokens = tokens
        self.asked = 0

    def result(self):
        self.asked += 1
        return self._tokens


class StubExecutor:
    """`deferred`: tokens come back as futures and the last one of a request is fed forward as
    -1, the way an executor does that leaves sampled tokens on the device."""

    def __init__(self, manager: CacheManager, deferred: bool = False) -> None:
        self.manager = manager
        self.deferred = deferred
        self.last: dict = {}
        self.calls = 0
        self.batches: list[list[tuple[str, int, int]]] = []   # per call: (request, start, count)

    def begin(self, key) -> bool:
        return self.manager.create_request(key) is not None

    def reserve(self, key, num_tokens):
        return self.manager.reserve(key, num_tokens)

    def release(self, key) -> int:
        return self.manager.free_request(key)

    def execute(self, work, record_logits):
        self.calls += 1
        self.batches.append([(w.seq.request_id, w.start, len(w.token_ids)) for w in work])
        results, tokens = [], []
        later = _Later(tokens)
        for w in work:
            key = w.seq.request_id
            assert w.start == self.manager.num_computed(key), "a portion must start where the cache ends"
            assert w.start + len(w.token_ids) <= self.manager.num_reserved(key), "tokens run without reserved room"
            assert list(w.token_ids) == w.seq.history[w.start : w.start + len(w.token_ids)]
            assert all(t >= 0 for t in w.token_ids[:-1]) or not w.wants_token or len(w.token_ids) == 1, "only the last token of a portion may be fed forward"
            self.manager.advance(key, len(w.token_ids))
            if w.wants_token:
                assert w.start + len(w.token_ids) == w.seq.history_len
                last = w.token_ids[-1]
                if last < 0:
                    assert self.deferred and key in self.last, "a token is fed forward that was never sampled"
                    last = self.last[key]
                token = next_token(last, w.start + len(w.token_ids) - 1)
                self.last[key] = token
                if self.deferred:
                    results.append(WorkResult(None, None, later, len(tokens)))
                    tokens.append(token)
                else:
                    results.append(WorkResult(token))
            else:
                results.append(WorkResult(None))
        return results
