"""The scheduler: admits requests, cuts prompts into portions, decodes, finishes, frees.

One decision per step (``plan``), pure host bookkeeping over the cache manager's counts:

1. Every running request that stands on a sampled token gets its one row first - decode
   before prompts is the reference's fairness rule
   (crates/shiso-runtime/src/scheduler/batching.rs:3-11).
2. What is left of the token budget (``max_num_batched_tokens``) goes to prompt portions:
   running requests still reading their prompt, oldest first, then waiting requests in
   arrival order while a sequence slot, a state slot and pages for all of the request's
   tokens so far are free.
   A portion is at most ``prefill_chunk`` tokens and may end anywhere, unless the model's plan
   names a ``portion_multiple``: then every portion but a request's last is a multiple of it
   (the reference's prefill grid, crates/shiso-runtime/src/scheduler/config.rs:35-44).  (The reference gives
   one prompt portion per tick to the oldest prefilling sequence only, batching.rs:219-227,
   and never mixes it with the decode pass; here both share one step.)
3. When a decode row cannot get a page: with ``on_exhaustion = "preempt"`` the youngest
   running request loses its cache and goes back to the head of the queue, to be recomputed
   from its tokens later (sampling depends only on logits, seed and position, so it
   continues with the same tokens); with ``"fail"`` the request that cannot grow ends with
   an error, which is what the reference does (crates/shiso-engine/src/kv.rs:597-609;
   crates/shiso-runtime/src/scheduler/mod.rs:2060-2063,2162-2168 - a resident session is
   never evicted there, scheduler/config.rs:276-283).  A request that cannot get a page
   although nothing else is left to preempt ends with an error in both modes.

A step's bookkeeping comes in two halves, so that the host need not wait for a step's tokens
before it plans the next one.  ``launched(plan)`` counts the step's tokens as computed and
puts a placeholder where each sampled token will go; a request that stands on a placeholder
can be planned again (its decode row then takes the token on the device, ``PlannedEntry.feed``);
one whose length budget the placeholder fills stops being planned (state ``draining``).
``arrived(plan, tokens)`` puts the values in: a stop token ends the request there, and what a
later step computed for it by then is dropped.  ``step_done`` is both at once.

Finishing (crates/shiso-runtime/src/scheduler/lifecycle.rs:1136-1208): a stop token ends the
request with reason ``stop`` (the token is counted, not emitted); ``max_new_tokens`` or the
context limit ends it with ``length``; ``abort`` ends it at once.  The budget at admission is
``min(max_new_tokens, ctx - prompt_len)`` (scheduler/mod.rs:1176-1179); a prompt that leaves
no room is refused up front.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Optional, Sequence

from ..sampling.params import SamplingParams

WAITING, RUNNING, DRAINING, FINISHED = "waiting", "running", "draining", "finished"
PENDING = -1  # stands in ``Request.output`` for a token that was sampled but has not reached the host


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 4
    max_num_batched_tokens: int = 2048
    prefill_chunk: Optional[int] = None  # longest prompt portion; None: the token budget
    ctx: int = 4096
    on_exhaustion: str = "preempt"  # or "fail"
    portion_multiple: int = 1  # portions that are not a request's last are multiples of this

    def __post_init__(self):
        if self.portion_multiple < 1:
            raise ValueError("portion_multiple must be at least 1")
        if self.portion_multiple > 1:
            room = min(self.max_num_batched_tokens - (self.max_num_seqs - 1), self.prefill_chunk or self.max_num_batched_tokens)
            if room < self.portion_multiple:
                raise ValueError(
                    f"portion_multiple = {self.portion_multiple}: beside {self.max_num_seqs - 1} decoding rows a step of "
                    f"{self.max_num_batched_tokens} tokens (prefill_chunk {self.prefill_chunk}) leaves {room} tokens, so a "
                    f"prompt could never advance"
                )
        if self.on_exhaustion not in ("preempt", "fail"):
            raise ValueError(f"on_exhaustion = {self.on_exhaustion!r}: expected 'preempt' or 'fail'")
        if self.max_num_seqs <= 0 or self.max_num_batched_tokens <= 0:
            raise ValueError("max_num_seqs and max_num_batched_tokens must be positive")
        if self.prefill_chunk is not None and self.prefill_chunk <= 0:
            raise ValueError("prefill_chunk must be positive")


@dataclass
class Request:
    id: object
    prompt: list
    params: SamplingParams
    stop_ids: frozenset = frozenset()
    output: list = field(default_factory=list)
    state: str = WAITING
    computed: int = 0  # tokens of prompt + output whose state is in the cache
    budget: int = 0  # most tokens it may still produce, fixed at admission
    finish_reason: Optional[str] = None
    error: Optional[str] = None
    preemptions: int = 0
    arrival: int = 0
    pending_row: Optional[int] = None  # which of the last step's sampling rows holds its pending token
    extras: Optional[dict] = None  # further per-row inputs of the prompt: name -> one int per prompt token

    def extras_slice(self, start: int, count: int) -> Optional[dict]:
        """The further per-row inputs of ``tokens[start : start + count]``: the prompt's own values,
        and the position for every token the request produced itself."""
        if not self.extras:
            return None
        n = len(self.prompt)
        return {name: [values[p] if p < n else p for p in range(start, start + count)] for name, values in self.extras.items()}

    @property
    def tokens(self) -> list:
        return self.prompt + self.output

    def token_slice(self, start: int, count: int) -> list:
        """``tokens[start : start + count]`` without joining prompt and output."""
        n = len(self.prompt)
        if start >= n:
            return self.output[start - n : start - n + count]
        if start + count <= n:
            return self.prompt[start : start + count]
        return self.prompt[start:] + self.output[: start + count - n]

    @property
    def remaining(self) -> int:
        return len(self.prompt) + len(self.output) - self.computed

    @property
    def decoding(self) -> bool:
        return self.state == RUNNING and self.remaining == 1 and len(self.output) > 0


@dataclass
class PlannedEntry:
    request: Request
    start: int  # index of the first token in request.tokens
    count: int
    samples: bool  # the portion reaches the request's last token: its logits are wanted
    feed: Optional[int] = None  # the one token is pending: the device takes it from this sampling row of the last step
    output_index: int = -1  # set by ``launched``: where in request.output the sampled token goes


@dataclass
class StepPlan:
    entries: list = field(default_factory=list)
    preempted: list = field(default_factory=list)
    failed: list = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(e.count for e in self.entries)


class Scheduler:
    def __init__(self, cache, config: SchedulerConfig, eos_token_ids: Sequence[int] = ()):
        self.cache = cache
        self.config = config
        self.eos = frozenset(eos_token_ids)
        self.waiting: deque = deque()
        self.running: list = []
        self.finished: list = []
        self._arrivals = 0
        self.stats = {"admitted": 0, "preempted": 0, "failed": 0, "finished": 0, "steps": 0,
                      "prefill_tokens": 0, "decode_tokens": 0}

    # ------------------------------------------------------------------ requests

    def add(self, request_id, prompt: Sequence[int], params: SamplingParams, extras: Optional[dict] = None) -> Request:
        prompt = [int(t) for t in prompt]
        stop = frozenset(int(t) for t in params.stop_token_ids)
        if not params.ignore_eos:
            stop = stop | self.eos
        req = Request(request_id, prompt, params, stop, arrival=self._arrivals)
        self._arrivals += 1
        if extras:
            req.extras = {name: [int(v) for v in values] for name, values in extras.items()}
            for name, values in req.extras.items():
                if len(values) != len(prompt):
                    return self._refuse(req, f"{len(values)} values of {name!r} for a prompt of {len(prompt)} tokens")
        if not prompt:
            return self._refuse(req, "empty prompt")
        if len(prompt) >= self.config.ctx:
            return self._refuse(req, f"prompt of {len(prompt)} tokens leaves no room in a context of {self.config.ctx}")
        if -(-len(prompt) // self.cache.page_size) > min(self.cache.max_blocks, self.cache.num_pages):
            return self._refuse(req, f"prompt of {len(prompt)} tokens does not fit the cache pool")
        req.budget = min(params.max_new_tokens, self.config.ctx - len(prompt))
        if req.budget <= 0:
            req.state, req.finish_reason = FINISHED, "length"
            self.finished.append(req)
            return req
        self.waiting.append(req)
        return req

    def _refuse(self, req: Request, why: str) -> Request:
        req.state, req.finish_reason, req.error = FINISHED, "error", why
        self.finished.append(req)
        self.stats["failed"] += 1
        return req

    def abort(self, request_id) -> bool:
        for req in list(self.running):
            if req.id == request_id:
                self._retire(req, "abort")
                return True
        for req in list(self.waiting):
            if req.id == request_id:
                self.waiting.remove(req)
                req.state, req.finish_reason = FINISHED, "abort"
                self.finished.append(req)
                return True
        return False

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def take_finished(self) -> list:
        done, self.finished = self.finished, []
        return done

    # ------------------------------------------------------------------ planning

    def plan(self) -> StepPlan:
        cfg = self.config
        plan = StepPlan()
        budget = cfg.max_num_batched_tokens
        chunk = cfg.prefill_chunk or cfg.max_num_batched_tokens
        free = list(self.cache.free_pages())
        free_slots = self.cache.slots.free_slots

        def fits(req, count):
            need = self.cache.pages_needed(req.id, count)
            return all(n <= f for n, f in zip(need, free)), need

        def claim(need):
            for g, n in enumerate(need):
                free[g] -= n

        # 1. decode rows, oldest first
        for req in list(self.running):
            if req.state != RUNNING or not req.decoding or budget <= 0:
                continue
            ok, need = fits(req, 1)
            while not ok:
                victim = self._victim(req, plan)
                alone = len([r for r in self.running if r.state == RUNNING]) <= 1
                if cfg.on_exhaustion == "fail" or victim is None or alone:
                    self._fail(req, "kv pool: no free page for the next position", plan)
                else:
                    self._preempt(victim, plan)
                # pages came back; those promised earlier in this plan stay promised
                free = list(self.cache.free_pages())
                for e in plan.entries:
                    claim(self.cache.pages_needed(e.request.id, e.count))
                free_slots = self.cache.slots.free_slots
                if req.state != RUNNING:
                    break
                ok, need = fits(req, 1)
            if req.state != RUNNING:
                continue
            claim(need)
            feed = req.pending_row if req.output[-1] == PENDING else None
            plan.entries.append(PlannedEntry(req, req.computed, 1, True, feed))
            budget -= 1

        # 2. prompt portions of running requests, oldest first
        for req in self.running:
            if (req.state != RUNNING or req.decoding or req.remaining <= 0 or budget <= 0
                    or any(e.request is req for e in plan.entries)):
                continue
            count = self._on_grid(req, self._portion(req, min(req.remaining, budget, chunk), free))
            if count <= 0:
                continue
            claim(self.cache.pages_needed(req.id, count))
            plan.entries.append(PlannedEntry(req, req.computed, count, count == req.remaining))
            budget -= count

        # 3. admissions in arrival order
        # (not in a step that had to preempt: the pages just freed are for the residents)
        while (self.waiting and budget > 0 and len(self.running) < cfg.max_num_seqs and free_slots > 0
               and not plan.preempted):
            req = self.waiting[0]
            # Pages for everything the request has so far must be free, not just for this
            # portion: a request admitted on less would soon be preempted again.
            if not fits(req, req.remaining)[0]:
                break
            count = self._on_grid(req, min(req.remaining, budget, chunk))
            if count <= 0:
                break  # what is left of this step's budget is less than one grid cell
            self.waiting.popleft()
            req.state = RUNNING
            self.running.append(req)
            self.stats["admitted"] += 1
            free_slots -= 1
            claim(self.cache.pages_needed(req.id, count))
            plan.entries.append(PlannedEntry(req, req.computed, count, count == req.remaining))
            budget -= count

        residents = [r for r in self.running if r.state == RUNNING]
        draining = len(residents) < len(self.running)  # those give their pages back by themselves
        if not plan.entries and residents and not draining and not plan.preempted and not plan.failed:
            # Residents but no work: nothing can ever free a page for them.  Fail the
            # youngest rather than spin (crates/shiso-runtime/src/scheduler/mod.rs:2148-2159).
            if len(residents) > 1 and cfg.on_exhaustion == "preempt":
                self._preempt(residents[-1], plan)
            else:
                self._fail(residents[-1], "kv pool: no request can make progress", plan)
        return plan

    def _on_grid(self, req: Request, count: int) -> int:
        """``count`` cut down to the plan's grid unless the portion reaches the request's last token."""
        multiple = self.config.portion_multiple
        if multiple > 1 and count < req.remaining:
            count -= count % multiple
        return count

    def _portion(self, req: Request, want: int, free) -> int:
        """The longest portion <= want whose pages are free now (0 when not even one token fits)."""
        if want <= 0:
            return 0
        need = self.cache.pages_needed(req.id, want)
        if all(n <= f for n, f in zip(need, free)):
            return want
        held = self.cache.length(req.id) if self.cache.has(req.id) else 0
        page = self.cache.page_size
        # tokens that fit into the pages the request holds plus the free ones of the scarcest group
        room = -(-held // page) * page - held + min(free) * page if free else want
        return max(0, min(want, room))

    def _victim(self, needy: Request, plan: StepPlan) -> Optional[Request]:
        """The youngest running request (the needy one itself when it is the youngest)."""
        candidates = [r for r in self.running if r.state == RUNNING]
        return candidates[-1] if candidates else None

    def _preempt(self, req: Request, plan: StepPlan) -> None:
        plan.entries = [e for e in plan.entries if e.request is not req]
        if self.cache.has(req.id):
            self.cache.release(req.id)
        self.running.remove(req)
        req.state, req.computed, req.pending_row = WAITING, 0, None
        req.preemptions += 1
        self.waiting.appendleft(req)
        plan.preempted.append(req)
        self.stats["preempted"] += 1

    def _fail(self, req: Request, why: str, plan: StepPlan) -> None:
        plan.entries = [e for e in plan.entries if e.request is not req]
        req.error = why
        self._retire(req, "error")
        plan.failed.append(req)
        self.stats["failed"] += 1

    def _retire(self, req: Request, reason: str) -> None:
        if self.cache.has(req.id):
            self.cache.release(req.id)
        if req in self.running:
            self.running.remove(req)
        if req in self.waiting:
            self.waiting.remove(req)
        req.state, req.finish_reason = FINISHED, reason
        self.finished.append(req)
        self.stats["finished"] += 1

    # ------------------------------------------------------------------ after the step

    def fail_step(self, plan: StepPlan, why: str) -> list:
        """The step did not run, or what it computed is not valid: its requests end with reason
        ``error`` and give their cache back; every other request goes on.  This is what the
        reference does with a pass that fails (crates/shiso-runtime/src/scheduler/mod.rs:1918-1927).
        Tokens that were sampled but never reached the host are dropped.  Returns the requests
        that ended."""
        failed = []
        for entry in plan.entries:
            req = entry.request
            if req.state == FINISHED:
                continue
            while req.output and req.output[-1] == PENDING:
                req.output.pop()
            req.pending_row = None
            req.error = why
            self._retire(req, "error")
            self.stats["failed"] += 1
            failed.append(req)
        return failed

    def launched(self, plan: StepPlan) -> None:
        """The step is on its way: its tokens count as computed, and a placeholder stands where
        each sampled token will go."""
        self.stats["steps"] += 1
        row = 0
        for entry in plan.entries:
            req = entry.request
            req.computed += entry.count
            if entry.count == 1 and req.output:
                self.stats["decode_tokens"] += 1
            else:
                self.stats["prefill_tokens"] += entry.count
            if not entry.samples:
                continue
            if req.state == RUNNING:
                assert req.remaining == 0, "a request is either reading its prompt or standing on a sampled token"
                entry.output_index = len(req.output)
                req.output.append(PENDING)
                req.pending_row = row
                if len(req.output) >= req.budget:
                    req.state = DRAINING  # nothing more to compute; it ends when the token arrives
            row += 1

    def arrived(self, plan: StepPlan, sampled: Sequence[int]) -> list:
        """``sampled[i]`` is the token picked for the i-th entry of the plan that samples.
        Returns the requests that finished with it."""
        done = []
        at = 0
        for entry in plan.entries:
            if not entry.samples:
                continue
            token = int(sampled[at])
            at += 1
            req, idx = entry.request, entry.output_index
            # a request that ended meanwhile (a stop token a step earlier, an abort, an error)
            # has no use for the token; one that was preempted still takes it
            if req.state == FINISHED or idx < 0 or idx >= len(req.output) or req.output[idx] != PENDING:
                continue
            if idx == len(req.output) - 1:
                req.pending_row = None
            if token in req.stop_ids:
                extra = len(req.output) - idx - 1  # computed past the stop before it was known
                del req.output[idx:]
                req.computed -= extra
                self._retire(req, "stop")
                done.append(req)
                continue
            req.output[idx] = token
            if req.state == DRAINING and idx == len(req.output) - 1:
                self._retire(req, "length")
                done.append(req)
        if at != len(sampled):
            raise ValueError(f"{len(sampled)} sampled tokens for {at} sampling entries")
        return done

    def step_done(self, plan: StepPlan, sampled: Sequence[int]) -> list:
        """Both halves at once, for a caller that waits for each step's tokens."""
        self.launched(plan)
        return self.arrived(plan, sampled)
