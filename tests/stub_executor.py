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


class StubExecutor:
    def __init__(self, manager: CacheManager) -> None:
        self.manager = manager
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
        results = []
        for w in work:
            key = w.seq.request_id
            assert w.start == self.manager.num_computed(key), "a portion must start where the cache ends"
            assert w.start + len(w.token_ids) <= self.manager.num_reserved(key), "tokens run without reserved room"
            assert list(w.token_ids) == w.seq.history[w.start : w.start + len(w.token_ids)]
            self.manager.advance(key, len(w.token_ids))
            if w.wants_token:
                assert w.start + len(w.token_ids) == w.seq.history_len
                results.append(WorkResult(next_token(w.token_ids[-1], w.start + len(w.token_ids) - 1)))
            else:
                results.append(WorkResult(None))
        return results
