"""The scheduler: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees.

One step = every runnable decode (at most ``max_decoding_seqs``) **plus** prompt portions
that fill what is left of ``max_num_batched_tokens`` (the reference runs either kind per
step, src/sparseengine/engine/scheduler.py:537-542; its chunking, budget and finish rules
are kept: :245-297, :1100-1160).  Capacity is counted in pages.

Admission: a waiting prompt is admitted when a row is free, fewer than
``max_num_seqs_in_gpu`` requests are resident, fewer than ``max_decoding_seqs`` are
decoding, and the pages for its **whole** prompt are free after setting aside what the
other unfinished prompts still need and a reservation for the tokens resident requests
will still produce (src/sparseengine/engine/scheduler.py:735-858).
Otherwise it waits, first come first served.

When pages run out while decoding: the request admitted last is **preempted** — its
pages and row are freed and it returns to the front of the waiting queue with its prompt
and the tokens it has produced; when readmitted it prefills all of them again and goes
on (recompute, cf. src/sparseengine/engine/scheduler.py:336-424).  Because sampling noise is
keyed by (request, number of produced tokens), the continuation draws the same noise; its
logits are those of a prompt step over the recomputed tokens instead of decode steps, equal up to
rounding, so a sampled token changes only where the draw falls on the edge between two tokens
(measured in bfloat16: one token in about 2,000).  A single
request that cannot take one more token with the whole cache to itself is an error, not
a loop.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from .sequence import Sequence, Status


@dataclass
class Planned:
    seq: Sequence
    start: int          # position of the portion's first token
    n_tokens: int
    samples: bool       # the portion reaches the request's last token: a token is sampled


@dataclass
class StepPlan:
    items: list = field(default_factory=list)
    preempted: list = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(i.n_tokens for i in self.items)

    @property
    def num_decodes(self) -> int:
        return sum(1 for i in self.items if i.seq.in_decode)


class Scheduler:
    def __init__(self, config, cache, eos_token_ids=(), max_model_len: int | None = None):
        self.config = config
        self.cache = cache
        self.eos_token_ids = frozenset(int(t) for t in eos_token_ids)
        self.max_model_len = int(max_model_len or cache.max_seq_len)
        self.waiting: deque = deque()
        self.running: list = []            # in admission order
        self.num_preemptions = 0

    # ---- queue -------------------------------------------------------------------------
    def add(self, seq: Sequence) -> None:
        if not seq.prompt_ids:
            raise ValueError("a request needs at least one prompt token")
        if len(seq.prompt_ids) + seq.params.max_tokens > self.max_model_len:
            raise ValueError(f"prompt ({len(seq.prompt_ids)} tokens) + max_tokens ({seq.params.max_tokens}) "
                             f"exceeds max_model_len ({self.max_model_len})")
        if self.cache.pages_for_tokens(len(seq.prompt_ids) + 1) > min(g.pool.num_pages for g in self.cache.groups):
            raise ValueError(f"a prompt of {len(seq.prompt_ids)} tokens does not fit the cache "
                             f"({min(g.pool.num_pages for g in self.cache.groups)} pages of {self.cache.page_size})")
        seq.status = Status.WAITING
        self.waiting.append(seq)

    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    def abort(self, seq_id) -> bool:
        for s in list(self.running):
            if s.seq_id == seq_id:
                self._drop(s, "abort")
                return True
        for s in list(self.waiting):
            if s.seq_id == seq_id:
                self.waiting.remove(s)
                s.status, s.finish_reason = Status.FINISHED, "abort"
                return True
        return False

    # ---- one step ----------------------------------------------------------------------
    def schedule(self) -> StepPlan:
        cfg = self.config
        plan = StepPlan()
        budget = cfg.max_num_batched_tokens
        wants: list = []

        decoders = [s for s in self.running if s.in_decode][: cfg.max_decoding_seqs]
        while decoders and not self.cache.can_reserve([(s.seq_id, 1) for s in decoders]):
            if len(self.running) == 1:
                raise RuntimeError(
                    f"request {self.running[0].seq_id} cannot take one more token although it has the whole "
                    f"cache ({self.cache.groups[0].pool.num_pages} pages of {self.cache.page_size}); "
                    "the cache is too small for this request")
            victim = self.running[-1]
            self._preempt(victim)
            plan.preempted.append(victim)
            decoders = [s for s in decoders if s is not victim]
        for s in decoders[:budget]:
            plan.items.append(Planned(s, s.num_computed, 1, True))
            wants.append((s.seq_id, 1))
        budget -= len(plan.items)

        portions = 0
        # unfinished prompts already resident go first, in admission order
        for s in self.running:
            if s.in_decode or s.remaining <= 0 or any(p.seq is s for p in plan.items):
                continue
            if portions >= cfg.max_num_seqs_in_batch or budget <= 0:
                break
            n = self._fit(s, min(s.remaining, cfg.engine_prefill_chunk_size, budget), wants)
            if n <= 0:
                continue
            plan.items.append(Planned(s, s.num_computed, n, n == s.remaining))
            wants.append((s.seq_id, n))
            budget -= n
            portions += 1

        # then new prompts, first come first served
        while (self.waiting and budget > 0 and portions < cfg.max_num_seqs_in_batch
               and not plan.preempted
               and self.cache.free_rows > 0 and len(self.running) < cfg.max_num_seqs_in_gpu
               and sum(1 for s in self.running if s.in_decode) < cfg.max_decoding_seqs):
            s = self.waiting[0]
            if not self._whole_prompt_fits(s, wants):
                break
            self.waiting.popleft()
            self.cache.admit(s.seq_id)
            s.status = Status.RUNNING
            self.running.append(s)
            n = min(s.remaining, cfg.engine_prefill_chunk_size, budget)
            plan.items.append(Planned(s, s.num_computed, n, n == s.remaining))
            wants.append((s.seq_id, n))
            budget -= n
            portions += 1

        if not plan.items and (self.waiting or self.running):
            if not self.running:
                s = self.waiting[0]
                raise RuntimeError(
                    f"request {s.seq_id} ({s.num_tokens} tokens) can never be admitted: the cache has "
                    f"{self.cache.groups[0].pool.num_pages} pages of {self.cache.page_size} tokens")
            raise RuntimeError("no runnable work although requests are resident")
        return plan

    def _fit(self, s: Sequence, n: int, wants: list) -> int:
        """Largest portion <= n whose pages are free beside what ``wants`` already takes."""
        while n > 0 and not self.cache.can_reserve(wants + [(s.seq_id, n)]):
            # drop to the end of the previous page
            filled = s.num_computed + n
            n = (filled - 1) // self.cache.page_size * self.cache.page_size - s.num_computed
        return max(n, 0)

    def _whole_prompt_fits(self, s: Sequence, wants: list) -> bool:
        """Pages for the whole of ``s``'s prompt, beside what this step already takes, what
        resident prompts still have to prefill and a reservation of
        ``decode_reservation_tokens`` future tokens per resident request
        (src/sparseengine/engine/cache_manager/decode_reservation.py:45-110)."""
        promised = list(wants)
        planned = dict(wants)
        for r in self.running:
            rest = 0 if r.in_decode else max(r.remaining - planned.get(r.seq_id, 0), 0)
            future = min(self.config.decode_reservation_tokens, r.params.max_tokens - len(r.output_ids))
            if rest + future > 0:
                promised.append((r.seq_id, rest + max(future, 0)))
        promised.append((s.seq_id, s.remaining + 1))
        return self.cache.can_reserve(promised)

    def _preempt(self, s: Sequence) -> None:
        self.cache.release(s.seq_id)
        self.running.remove(s)
        s.num_computed = 0
        s.status = Status.WAITING
        s.preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(s)

    def _drop(self, s: Sequence, reason: str) -> None:
        if self.cache.has(s.seq_id):
            self.cache.release(s.seq_id)
        if s in self.running:
            self.running.remove(s)
        s.status, s.finish_reason = Status.FINISHED, reason

    def fail(self, plan: StepPlan, reason: str = "error") -> list:
        """The step of ``plan`` gave no usable result: every request of it that still runs is
        ended with ``reason`` and gives its pages and its row back.  Returns those requests."""
        ended = []
        for item in plan.items:
            if item.seq.status == Status.RUNNING:
                self._drop(item.seq, reason)
                ended.append(item.seq)
        return ended

    # ---- after the step ----------------------------------------------------------------
    def postprocess(self, plan: StepPlan, tokens: list, logprobs=None, top_logprobs=None) -> list:
        """``tokens``: one sampled token per planned item that samples, in plan order.
        Returns the requests that finished."""
        finished = []
        it = iter(range(len(tokens)))
        for item in plan.items:
            s = item.seq
            if s.status != Status.RUNNING:       # ended (or was preempted) while this step was on its way:
                if item.samples:                 # its token is one too many
                    next(it)
                continue
            s.num_computed += item.n_tokens
            if not item.samples:
                continue
            i = next(it)
            forced = s.params.benchmark_forced_token_ids
            tok = int(forced[len(s.output_ids)]) if forced is not None else int(tokens[i])
            s.output_ids.append(tok)
            if logprobs is not None:
                s.logprobs.append(logprobs[i])
            if top_logprobs is not None:
                s.top_logprobs.append(top_logprobs[i])
            eos = s.params.eos_token_ids or self.eos_token_ids
            if not s.params.ignore_eos and tok in eos:
                reason = "stop"
            elif len(s.output_ids) >= s.params.max_tokens or s.num_tokens >= self.max_model_len:
                reason = "length"
            else:
                continue
            self._drop(s, reason)
            finished.append(s)
        return finished
