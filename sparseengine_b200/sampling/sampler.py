"""The sampler: next tokens from logits rows, on the device (kernels: csrc/sampling.cu).

Greedy, temperature, top-k, top-p, presence and repetition penalties, optional
log-probabilities — what the reference samples with (src/sparseengine/layers/sampler.py:5-142,
src/sparseengine/engine/model_runner.py:2528-2569).  Unlike the reference's process-global
generator, every row draws from its own counter-based stream keyed by
(sampler seed, request id, number of tokens the request has produced), so a request's
tokens do not depend on batch composition, chunking or preemption.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import Sequence

import numpy as np
import torch

from ..csrc import ops_sampling as sops
from .params import SamplingParams


@dataclass
class SampleRequest:
    params: SamplingParams
    seq_id: object
    step: int                                   # tokens produced so far by this request
    prompt_ids: Sequence[int] = ()
    output_ids: Sequence[int] = ()


def row_seed(sampler_seed: int, seq_id, step: int) -> int:
    h = hashlib.blake2b(f"{sampler_seed}|{seq_id!r}|{step}".encode(), digest_size=8).digest()
    return int.from_bytes(h, "little")


class _PinnedPool:
    """Pinned host buffers for results on their way back, reused (allocating one is slow)."""

    def __init__(self):
        self.free: dict = {}

    def take(self, n: int, dtype) -> torch.Tensor:
        size = 1 << max(6, (max(n, 1) - 1).bit_length())
        lst = self.free.setdefault((size, dtype), [])
        return lst.pop() if lst else torch.empty(size, dtype=dtype, pin_memory=True)

    def give(self, t: torch.Tensor) -> None:
        self.free.setdefault((t.numel(), t.dtype), []).append(t)


class Pending:
    """What :meth:`Sampler.submit` queued: the tokens (and log-probabilities) of one step on
    their way to pinned host memory, and an event that says when they have arrived.
    ``tokens_device`` are the sampled ids on the device (int32 ``[n]``), for a next step that is
    launched before the host has seen them."""

    def __init__(self):
        self.tokens_device = None
        self.event = None
        self.n = 0
        self.requests = ()
        self.host = {}           # name -> (pinned buffer, shape)
        self.keep = []           # device tensors that must outlive the copies
        self.top_rows = []
        self.top_n = 0


class Sampler:
    def __init__(self, seed: int = 0):
        self.seed = int(seed)
        # per row of the last call: {token id: log-probability} of the most likely tokens for
        # requests with logprobs = n > 0 (src/sparseengine/engine/model_runner.py:2528-2569), else None
        self.last_top_logprobs = None
        self._pool = _PinnedPool()

    def _upload(self, host: np.ndarray, dev) -> torch.Tensor:
        """A small host array to the device through pinned memory, without blocking the host."""
        pin = self._pool.take(host.size, torch.int32)
        pin[:host.size].numpy()[:] = host.view(np.int32)
        d = torch.empty(host.size, dtype=torch.int32, device=dev)
        d.copy_(pin[:host.size], non_blocking=True)
        return d, pin

    def submit(self, logits: torch.Tensor, requests: Sequence[SampleRequest]) -> Pending:
        """Queue the sampling of every row and the copies of the results to the host; nothing
        here waits for the device."""
        n, vocab = logits.shape
        if n != len(requests):
            raise ValueError("one sampling request per logits row is needed")
        dev = logits.device
        pend = Pending()
        pend.n, pend.requests = n, list(requests)
        want_lp = any(r.params.logprobs is not None for r in requests)
        out = torch.empty(n, dtype=torch.int32, device=dev)
        lp = torch.empty(n, dtype=torch.float32, device=dev) if want_lp else None
        pins = []

        if any(r.params.has_penalties for r in requests):
            logits = self._penalised(logits, requests)

        if all(r.params.greedy for r in requests):
            sops.sample(logits, None, None, None, None, out, lp)
        else:
            # one packed upload: seeds (2 words a row) first, then temperature, top-k, top-p
            host = np.empty(5 * n, dtype=np.uint32)
            f = host.view(np.float32)
            for i, r in enumerate(requests):
                s = row_seed(self.seed, r.seq_id, r.step)
                host[2 * i], host[2 * i + 1] = s & 0xFFFFFFFF, s >> 32
                f[2 * n + i] = r.params.temperature
                host[3 * n + i] = min(r.params.top_k, vocab)
                f[4 * n + i] = r.params.top_p
            d, pin = self._upload(host, dev)
            pins.append(pin)
            seeds = d[:2 * n].view(torch.int64)
            temp = d[2 * n:3 * n].view(torch.float32)
            top_k = d[3 * n:4 * n]
            top_p = d[4 * n:5 * n].view(torch.float32)
            if not any(0 < r.params.top_k < vocab or r.params.top_p < 1.0 for r in requests):
                top_k = top_p = None            # no cuts anywhere: the kernels with many blocks per row
            sops.sample(logits, temp, top_k, top_p, seeds, out, lp)
            pend.keep.append(d)
        # the n most likely tokens of the rows that asked for them (logprobs = n > 0)
        pend.top_rows = [i for i, r in enumerate(requests) if r.params.logprobs]
        pend.top_n = min(max((requests[i].params.logprobs for i in pend.top_rows), default=0), vocab)
        results = {"tokens": out}
        if want_lp:
            results["lp"] = lp
        if pend.top_rows:
            rows_d, pin = self._upload(np.asarray(pend.top_rows, dtype=np.int32), dev)
            pins.append(pin)
            top_ids = torch.empty(len(pend.top_rows), pend.top_n, dtype=torch.int32, device=dev)
            top_vals = torch.empty(len(pend.top_rows), pend.top_n, dtype=torch.float32, device=dev)
            sops.top_logprobs(logits, rows_d, top_ids, top_vals)
            results["top_ids"], results["top_vals"] = top_ids, top_vals
            pend.keep.append(rows_d)
        for name, t in results.items():
            pin = self._pool.take(t.numel(), t.dtype)
            pin[:t.numel()].copy_(t.reshape(-1), non_blocking=True)
            pend.host[name] = (pin, tuple(t.shape))
        pend.keep += list(results.values()) + [logits]
        pend.tokens_device = out
        pend.event = torch.cuda.Event()
        pend.event.record()
        pend._pins = pins
        return pend

    def collect(self, pend: Pending):
        """Wait for what :meth:`submit` queued; returns (tokens, logprobs or None, top log-probabilities or None)."""
        pend.event.synchronize()

        def host(name):
            pin, shape = pend.host[name]
            n = int(np.prod(shape)) if shape else 1
            return pin[:n].view(*shape).tolist() if len(shape) > 1 else pin[:n].tolist()
        tokens = host("tokens")
        logprobs = None
        if "lp" in pend.host:
            chosen = host("lp")
            logprobs = [chosen[i] if r.params.logprobs is not None else None for i, r in enumerate(pend.requests)]
        tops = None
        if pend.top_rows:
            ids_h, vals_h = host("top_ids"), host("top_vals")
            tops = [None] * pend.n
            for k, i in enumerate(pend.top_rows):
                want = min(pend.requests[i].params.logprobs, pend.top_n)
                tops[i] = {int(t): float(v) for t, v in zip(ids_h[k][:want], vals_h[k][:want]) if t >= 0}
        for pin, _ in pend.host.values():
            self._pool.give(pin)
        for pin in pend._pins:
            self._pool.give(pin)
        pend.host, pend.keep, pend._pins = {}, [], []
        return tokens, logprobs, tops

    def sample(self, logits: torch.Tensor, requests: Sequence[SampleRequest]):
        """logits [n, vocab] (activation dtype) → (token ids list[int], logprobs list or None)."""
        tokens, logprobs, tops = self.collect(self.submit(logits, requests))
        self.last_top_logprobs = tops
        return tokens, logprobs

    def _penalised(self, logits, requests):
        n, vocab = logits.shape
        dev = logits.device
        work = torch.empty(n, vocab, dtype=torch.float32, device=dev)
        sops.to_float(logits, work)
        pairs = []
        rep = np.ones(n, dtype=np.float32)
        pres = np.zeros(n, dtype=np.float32)
        for i, r in enumerate(requests):
            if not r.params.has_penalties:
                continue
            rep[i], pres[i] = r.params.repetition_penalty, r.params.presence_penalty
            completion = set(int(t) for t in r.output_ids)
            everything = completion | set(int(t) for t in r.prompt_ids)
            for t in everything:
                pairs.append((i, t, 1 | (2 if t in completion else 0)))
        if pairs:
            p = torch.tensor(pairs, dtype=torch.int32, device=dev).view(-1)
            sops.apply_penalties(work, p, len(pairs), torch.from_numpy(rep).to(dev), torch.from_numpy(pres).to(dev))
        return work
