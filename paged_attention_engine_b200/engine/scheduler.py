"""Continuous batching: every step decides what runs.

The decisions are the reference's (engine/scheduler.py:1-58,301-770), restated over this
engine's step function:

  1. Admit from the head of the waiting queue while the head fits: strict first come,
     first served, nothing behind a head that does not fit is looked at
     (engine/scheduler.py:496-518). A head fits when there are pages for its whole
     history with `admission_margin_blocks` left over in every pool
     (engine/scheduler.py:376-379), the running set is under `max_num_seqs`, and the
     step's token budget has room.
  2. Every other running request goes on: one decoded token, or the next portion of its
     prompt. A decode needs at most one new page per pool and may spend the margin
     (engine/scheduler.py:381-385).
  3. When a decode finds no page, the newest running requests are preempted until it
     does (engine/scheduler.py:624-674): a victim gives back everything, returns to the
     queue in arrival order, and is later recomputed from prompt + generated tokens,
     which yields exactly one new token (engine/scheduler.py:520-552).
  4. The step's work runs as ONE batch; a request that reaches `max_new_tokens` leaves
     and its pages go back when the step ends (the reference's fused mode,
     engine/scheduler.py:49-58). End-of-sequence tokens are ignored: a request yields
     exactly `max_new_tokens` tokens (engine/model.py:466-469).

A request that could never fit (prompt + max_new_tokens needs more pages than a pool
has, less the margin) is rejected when it is offered (engine/scheduler.py:423-449): let
in, it would evict itself for ever. Because every admitted request fits alone, the
victims of a preemption are never the whole running set.

What differs from the reference, by design of the step function: batches are not
padded, so `max_num_batched_tokens` bounds the tokens that really run
(the reference bounds rows x longest row, engine/scheduler.py:462-482), and a prompt
that is longer than what is left of the budget is cut: it runs as many tokens as fit
and goes on in the next step. Within the budget, one token is set aside for every
request that decodes, prompts under way come next, new admissions take the rest.
"""

from __future__ import annotations

import time
import zlib
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Hashable, Protocol, Sequence as Seq

from ..cache.allocator import AllocResult
from ..cache.manager import CacheManager

ADMISSION_MARGIN_BLOCKS = 1   # engine/cache.py:35 of the reference


class EventKind(Enum):
    ADMIT = "admit"
    FINISH = "finish"
    PREEMPT = "preempt"
    RECOMPUTE = "recompute"
    REJECT = "reject"


@dataclass(frozen=True)
class Event:
    """One decision with the pool's state at that moment (engine/scheduler.py:121-145)."""

    timestamp: float
    step: int
    kind: EventKind
    request_id: str
    detail: str
    free_blocks: int
    running: int
    waiting: int
    tokens_held: int = 0


@dataclass(frozen=True)
class Request:
    """What a user asks for. `temperature` 0 is greedy; `seed` makes a temperature draw
    repeatable (None: the engine's seed, 0 unless its options say otherwise)."""

    request_id: str
    prompt_token_ids: tuple[int, ...]
    max_new_tokens: int
    temperature: float = 0.0
    seed: int | None = None

    def __post_init__(self) -> None:
        object.__setattr__(self, "prompt_token_ids", tuple(int(t) for t in self.prompt_token_ids))
        if not self.prompt_token_ids:
            raise ValueError(f"{self.request_id}: prompt must be non-empty")
        if self.max_new_tokens < 1:
            raise ValueError(f"{self.request_id}: max_new_tokens must be at least 1")
        if self.temperature < 0.0:
            raise ValueError(f"{self.request_id}: temperature must not be negative")

    @property
    def prompt_len(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def max_total_len(self) -> int:
        return self.prompt_len + self.max_new_tokens

    @property
    def sampling_key(self) -> int:
        """A number that belongs to the request id alone; part of the sampler's counter."""
        return zlib.crc32(self.request_id.encode()) & 0x7FFFFFFF


class SequenceStatus(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"
    REJECTED = "rejected"


@dataclass
class Sequence:
    """A request's state while it lives; it survives preemption and readmission."""

    request: Request
    arrival_index: int
    generated: list[int] = field(default_factory=list)
    status: SequenceStatus = SequenceStatus.WAITING
    num_computed: int = 0          # tokens of the history whose keys and values are cached
    preemption_count: int = 0      # never read by a decision
    step_logits: list = field(default_factory=list)   # filled when record_logits is set

    @property
    def request_id(self) -> str:
        return self.request.request_id

    @property
    def history(self) -> list[int]:
        return list(self.request.prompt_token_ids) + self.generated

    @property
    def history_len(self) -> int:
        return self.request.prompt_len + len(self.generated)

    def history_slice(self, start: int, count: int) -> tuple[int, ...]:
        """Tokens start .. start + count - 1 of the history, without building all of it."""
        prompt = self.request.prompt_token_ids
        n = len(prompt)
        end = start + count
        if end <= n:
            return tuple(prompt[start:end])
        if start >= n:
            return tuple(self.generated[start - n : end - n])
        return tuple(prompt[start:]) + tuple(self.generated[: end - n])

    @property
    def is_finished(self) -> bool:
        return len(self.generated) >= self.request.max_new_tokens


@dataclass(frozen=True)
class ScheduledWork:
    """One request's share of a step: tokens at consecutive positions from `start`."""

    seq: Sequence
    token_ids: tuple[int, ...]
    start: int
    is_prefill: bool
    wants_token: bool       # False for a portion that ends before the history does


@dataclass(frozen=True)
class StepResult:
    step: int
    admitted: tuple[str, ...]
    decoded: tuple[str, ...]
    finished: tuple[str, ...]
    preempted: tuple[str, ...]
    running: int
    waiting: int
    free_blocks: int
    batch_size: int = 0
    deferred: tuple[str, ...] = ()
    batched_token_cost: int = 0            # tokens that ran in this step's batch
    prefilled: tuple[str, ...] = ()        # requests that ran a portion of their history


# What stands in `Sequence.generated` for a token that was sampled on the device and has
# not been read back yet. It is also what the step function takes for "the token this
# request sampled in the step before".
PENDING = -1


@dataclass
class WorkResult:
    """The token of one portion, or a `future` whose `result()[row]` will be that token: an
    executor may leave sampled tokens on the device and hand them over a step later, so that
    the host plans the next step while this one runs."""

    token: int | None
    logits: object = None
    future: object = None
    row: int = -1


class Executor(Protocol):
    """What the scheduler needs of a model (engine/scheduler.py:255-272): reservation is
    apart from execution because capacity is the scheduler's decision."""

    def begin(self, key: Hashable) -> bool: ...

    def reserve(self, key: Hashable, num_tokens: int) -> AllocResult: ...

    def release(self, key: Hashable) -> int: ...

    def execute(self, work: Seq[ScheduledWork], record_logits: bool) -> list[WorkResult]: ...


class Scheduler:
    def __init__(
        self,
        executor: Executor,
        cache_manager: CacheManager,
        admission_margin_blocks: int = ADMISSION_MARGIN_BLOCKS,
        clock: Callable[[], float] = time.monotonic,
        record_logits: bool = False,
        max_num_seqs: int | None = None,
        max_num_batched_tokens: int | None = None,
        max_model_len: int | None = None,
        pipeline_depth: int = 2,
    ) -> None:
        if admission_margin_blocks < 0:
            raise ValueError(f"admission_margin_blocks must not be negative, got {admission_margin_blocks}")
        if max_num_seqs is not None and max_num_seqs < 1:
            raise ValueError(f"max_num_seqs must be at least 1, got {max_num_seqs}")
        if max_num_batched_tokens is not None and max_num_batched_tokens < 1:
            raise ValueError(f"max_num_batched_tokens must be at least 1, got {max_num_batched_tokens}")
        self.executor = executor
        self.cache = cache_manager
        self.admission_margin_blocks = admission_margin_blocks
        self.clock = clock
        self.record_logits = record_logits
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_model_len = max_model_len
        # How many steps may be under way before the oldest one's tokens are read back (only
        # an executor that hands out futures makes use of it).
        self.pipeline_depth = max(1, pipeline_depth)

        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.finished: dict[str, Sequence] = {}
        self.rejected: dict[str, Sequence] = {}
        self.events: list[Event] = []
        self._step = 0
        self._next_arrival = 0
        self._plan: list[ScheduledWork] = []
        self._budget_left = 0
        self._unresolved: list[tuple[Sequence, int, object, int]] = []   # (sequence, index in generated, future, row)

    # -- log ---------------------------------------------------------------- #

    def _log(self, kind: EventKind, seq: Sequence, detail: str = "") -> None:
        self.events.append(
            Event(
                timestamp=self.clock(), step=self._step, kind=kind, request_id=seq.request_id, detail=detail,
                free_blocks=self.cache.num_free, running=len(self.running), waiting=len(self.waiting),
                tokens_held=self.cache.tokens_held(),
            )
        )

    def events_of(self, kind: EventKind) -> list[Event]:
        return [e for e in self.events if e.kind is kind]

    # -- intake ------------------------------------------------------------- #

    @property
    def max_admissible_blocks(self) -> int:
        return self.cache.num_blocks - self.admission_margin_blocks

    def add_request(self, request: Request) -> bool:
        """Offers a request; False when the admission guard rejects it."""
        seq = Sequence(request=request, arrival_index=self._next_arrival)
        self._next_arrival += 1
        reason = None
        if not self.cache.fits_alone(request.max_total_len, self.admission_margin_blocks):
            reason = (
                f"max length {request.max_total_len} needs {self.cache.blocks_needed(request.max_total_len)} blocks, "
                f"limit is {self.max_admissible_blocks} ({self.cache.num_blocks} - {self.admission_margin_blocks} margin)"
            )
        elif self.max_model_len is not None and request.max_total_len > self.max_model_len:
            reason = f"max length {request.max_total_len} exceeds the model's {self.max_model_len} positions"
        if reason is not None:
            seq.status = SequenceStatus.REJECTED
            self.rejected[request.request_id] = seq
            self._log(EventKind.REJECT, seq, reason)
            return False
        self.waiting.append(seq)
        return True

    # -- planning ----------------------------------------------------------- #

    def _plan_portion(self, seq: Sequence, is_prefill: bool) -> None:
        """Plans the next tokens of `seq`'s history: as many as the budget has room for."""
        pending = seq.history_len - seq.num_computed
        count = min(pending, self._budget_left)
        self._plan.append(
            ScheduledWork(
                seq=seq, token_ids=seq.history_slice(seq.num_computed, count),
                start=seq.num_computed, is_prefill=is_prefill, wants_token=count == pending,
            )
        )
        self._budget_left -= count

    def _admit(self) -> list[Sequence]:
        admitted: list[Sequence] = []
        while self.waiting:
            head = self.waiting[0]
            if self.max_num_seqs is not None and len(self.running) >= self.max_num_seqs:
                break
            if not self.cache.can_append(None, head.history_len, self.admission_margin_blocks):
                break
            if self._budget_left < 1:
                break
            self.waiting.popleft()
            self._start(head)
            admitted.append(head)
        return admitted

    def resolve(self, keep_steps: int = 0) -> None:
        """Reads back the sampled tokens that are still on the device, all but those of the
        newest `keep_steps` steps (waits for the steps it reads)."""
        futures = []
        for _, _, future, _ in self._unresolved:
            if not futures or futures[-1] is not future:
                futures.append(future)
        keep = set(id(f) for f in futures[len(futures) - keep_steps:]) if keep_steps > 0 else set()
        left = []
        for seq, index, future, row in self._unresolved:
            if id(future) in keep:
                left.append((seq, index, future, row))
            else:
                seq.generated[index] = int(future.result()[row])
        self._unresolved = left

    def _start(self, seq: Sequence) -> None:
        is_recompute = bool(seq.generated)
        if is_recompute and seq.generated[-1] == PENDING:
            self.resolve()        # a recompute replays the tokens themselves
        if not self.executor.begin(seq.request_id):
            raise AssertionError(f"{seq.request_id}: no state slot although the capacity check passed")
        seq.status = SequenceStatus.RUNNING
        seq.num_computed = 0
        self.running.append(seq)
        total = seq.history_len
        self._log(
            EventKind.ADMIT, seq,
            f"prefill {total} tokens" + (f", readmission #{seq.preemption_count}" if is_recompute else ""),
        )
        if is_recompute:
            self._log(
                EventKind.RECOMPUTE, seq,
                f"replaying {total} tokens ({seq.request.prompt_len} prompt + {len(seq.generated)} generated)",
            )
        self._reserve(seq, total)
        self._plan_portion(seq, is_prefill=True)

    def _reserve(self, seq: Sequence, count: int) -> None:
        result = self.executor.reserve(seq.request_id, count)
        if not result.ok:
            raise AssertionError(
                f"{seq.request_id}: reserving {count} token(s) failed with {result.status.value} "
                "after the capacity check passed"
            )

    def _evict(self, seq: Sequence) -> None:
        self.running.remove(seq)
        for work in self._plan:
            if work.seq is seq:
                self._budget_left += len(work.token_ids)
        self._plan = [w for w in self._plan if w.seq is not seq]
        freed = self.executor.release(seq.request_id)
        seq.status = SequenceStatus.WAITING
        seq.num_computed = 0
        seq.preemption_count += 1
        self._log(EventKind.PREEMPT, seq, f"freed {freed} blocks, {len(seq.generated)} generated tokens to replay")
        self.waiting.append(seq)
        self.waiting = deque(sorted(self.waiting, key=lambda s: s.arrival_index))

    def _make_room_for(self, seq: Sequence) -> list[Sequence]:
        """Preempts the newest running requests until `seq` can grow by one token, or
        until `seq` itself was the newest."""
        before = len(self.running)
        victims: list[Sequence] = []
        while not self.cache.can_append(seq.request_id, 1, 0):
            if not self.running:
                raise AssertionError(f"{seq.request_id}: nothing left to preempt and still no page")
            victim = max(self.running, key=lambda s: s.arrival_index)
            victims.append(victim)
            self._evict(victim)
            if victim is seq:
                break
        assert len(victims) < before, "the victims are the whole running set: the admission guard failed"
        return victims

    # -- one step ----------------------------------------------------------- #

    def step(self) -> StepResult:
        self._step += 1
        self._plan = []
        budget = self.max_num_batched_tokens if self.max_num_batched_tokens is not None else 1 << 60

        was_running = list(self.running)
        # A request whose history is one token longer than its reserved room decodes: it
        # has to grow. The others still have reserved tokens to run (a prompt under way).
        decoders = [s for s in was_running if s.history_len - self.cache.num_reserved(s.request_id) == 1]
        # One token is set aside for every request that decodes; if even that does not
        # fit, the oldest decode and the rest wait a step (they keep their pages).
        deferred: list[str] = []
        if len(decoders) > budget:
            deferred = [s.request_id for s in decoders[budget:]]
            decoders = decoders[:budget]
        decoder_ids = {id(s) for s in decoders}
        self._budget_left = budget - len(decoders)

        # Prompts under way come before new admissions.
        for seq in was_running:
            if id(seq) in decoder_ids or seq.request_id in deferred:
                continue
            if self._budget_left > 0 and seq.history_len - seq.num_computed > 0:
                self._plan_portion(seq, is_prefill=True)

        admitted = self._admit()

        preempted: list[str] = []
        finished_before = set(self.finished)
        for seq in decoders:
            if seq.status is not SequenceStatus.RUNNING:
                continue      # preempted earlier in this step
            if not self.cache.can_append(seq.request_id, 1, 0):
                victims = self._make_room_for(seq)
                preempted.extend(v.request_id for v in victims)
                if seq.status is not SequenceStatus.RUNNING:
                    continue  # it was its own victim
            self._reserve(seq, 1)
            self._budget_left += 1          # its token was set aside above
            self._plan_portion(seq, is_prefill=False)

        ran = self._flush()
        return StepResult(
            step=self._step,
            admitted=tuple(s.request_id for s in admitted),
            decoded=tuple(w.seq.request_id for w in ran if not w.is_prefill),
            finished=tuple(sorted(set(self.finished) - finished_before)),
            preempted=tuple(preempted),
            running=len(self.running),
            waiting=len(self.waiting),
            free_blocks=self.cache.num_free,
            batch_size=len(ran),
            deferred=tuple(deferred),
            batched_token_cost=sum(len(w.token_ids) for w in ran),
            prefilled=tuple(w.seq.request_id for w in ran if w.is_prefill),
        )

    def _flush(self) -> list[ScheduledWork]:
        """The step's one batch, then one new token for every portion that ended a history."""
        plan, self._plan = self._plan, []
        if not plan:
            return plan
        results = self.executor.execute(plan, self.record_logits)
        if len(results) != len(plan):
            raise AssertionError(f"the executor answered {len(results)} results for {len(plan)} portions")
        # This step is on its way; the tokens of older steps can be read now without leaving
        # the device idle (this step's own futures are appended below).
        self.resolve(keep_steps=self.pipeline_depth - 1)
        for work, result in zip(plan, results):
            seq = work.seq
            seq.num_computed += len(work.token_ids)
            if not work.wants_token:
                continue
            if self.record_logits:
                seq.step_logits.append(result.logits)
            if result.future is not None:
                seq.generated.append(PENDING)
                self._unresolved.append((seq, len(seq.generated) - 1, result.future, result.row))
            elif result.token is None:
                raise AssertionError(f"{seq.request_id}: no token for a portion that ended its history")
            else:
                seq.generated.append(int(result.token))
            if seq.is_finished:
                self._finish(seq)
        return plan

    def _finish(self, seq: Sequence) -> None:
        self.running.remove(seq)
        freed = self.executor.release(seq.request_id)
        seq.status = SequenceStatus.FINISHED
        self.finished[seq.request_id] = seq
        self._log(EventKind.FINISH, seq, f"{len(seq.generated)} tokens, freed {freed} blocks")

    def run_to_completion(self, max_steps: int = 100_000) -> dict[str, tuple[int, ...]]:
        """Steps until nothing waits or runs; {request_id: generated tokens}. `max_steps`
        is a backstop against a scheduler that makes no progress, not a policy
        (engine/scheduler.py:753-770)."""
        steps = 0
        while self.waiting or self.running:
            self.step()
            steps += 1
            if steps > max_steps:
                raise RuntimeError(
                    f"no progress after {max_steps} steps: {len(self.waiting)} waiting, {len(self.running)} running"
                )
        self.resolve()
        return {rid: tuple(seq.generated) for rid, seq in self.finished.items()}
