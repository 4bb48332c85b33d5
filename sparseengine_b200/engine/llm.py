"""The Python entry point, in the reference's manner
(src/sparseengine/llm.py:1-5, src/sparseengine/engine/llm_engine.py:232-348,872-1018,1754-2055):

    llm = LLM(model_folder, max_num_batched_tokens=8192, dtype="bfloat16", ...)
    outs = llm.generate([[1, 2, 3], "a string needs a tokenizer"], SamplingParams(temperature=0))
    outs[0]["token_ids"], outs[0]["text"]

``LLM(model, **options)`` takes the fields of :class:`Config` and refuses unknown names.
``generate`` returns ``[{"text", "token_ids"}]`` in the order of the prompts; ``add_request``
/ ``step`` / ``is_finished`` drive the engine by hand; ``step`` returns
``(finished outputs, num_tokens)`` with ``num_tokens > 0`` the prompt tokens of the step,
or ``-n`` for a step of ``n`` decoded tokens only.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Optional, Sequence as Seq

import torch

from ..config.engine_config import Config
from ..config.registry import read_config_json
from ..sampling.params import SamplingParams
from ..sampling.sampler import SampleRequest, Sampler
from .factory import build_runner, require_cuda, resolve_dtype
from .runner import StepEntry
from .scheduler import Scheduler
from .sequence import Sequence, Status


def _eos_from_folder(model_dir: str, raw: dict) -> tuple:
    """EOS ids from generation_config.json, else config.json
    (src/sparseengine/engine/llm_engine.py:206-222)."""
    for name in ("generation_config.json",):
        path = os.path.join(model_dir, name)
        if os.path.isfile(path):
            with open(path) as f:
                v = json.load(f).get("eos_token_id")
            if v is not None:
                return tuple(v) if isinstance(v, list) else (int(v),)
    v = raw.get("eos_token_id")
    if v is None:
        return ()
    return tuple(v) if isinstance(v, list) else (int(v),)


class _InFlight:
    """A step that has been queued on the device: its plan and its sampling results on their way."""

    def __init__(self, plan, pending):
        self.plan = plan
        self.pending = pending


class LLM:
    def __init__(self, model, **options):
        self.config = Config.from_kwargs(model, **options)
        cfg = self.config
        from .factory import check_kernel_tuning
        check_kernel_tuning(cfg.kernel_tuning)
        device = require_cuda(cfg.device)
        from ..csrc import ops
        ops.library()       # compile/load the kernels now; there is no other path
        raw = model if isinstance(model, dict) else read_config_json(model)
        raw = cfg.apply_tiny_random_overrides(raw)
        self._raw = raw
        dt = resolve_dtype(cfg.dtype)
        from ..config.registry import load_model_spec
        _, spec = load_model_spec(raw)
        self.max_model_len = min(cfg.max_model_len or spec.max_position, spec.max_position)
        random = cfg.tiny_random or isinstance(model, dict)
        # weights first; the cache is then sized from what they left
        self.runner = build_runner(
            raw if random else model, dtype=dt, page_size=cfg.page_size,
            num_pages=lambda m: self._num_pages(m, dt, device), max_rows=cfg.max_num_seqs_in_gpu,
            max_seq_len=self.max_model_len, device=device, random_weights=random, seed=cfg.tiny_random_seed,
            random_std=cfg.tiny_random_std, norm_std=cfg.tiny_random_norm_std, bias_std=cfg.tiny_random_bias_std,
            decode_graphs=cfg.decode_graph and not cfg.enable_profiler, state_slot_bytes=cfg.state_slot_bytes,
            mlp_chunk_size=cfg.mlp_chunk_size, kernel_tuning=cfg.kernel_tuning)
        cache = self.runner.cache
        self.runner.validate = cfg.validate_runtime_invariants
        self.runner.model.profile = {} if cfg.enable_profiler else None
        eos = tuple(cfg.eos_token_ids) or ((cfg.eos,) if cfg.eos >= 0 else ())
        if not eos and not isinstance(model, dict):
            eos = _eos_from_folder(model, raw)
        self.scheduler = Scheduler(cfg, cache, eos_token_ids=eos, max_model_len=self.max_model_len)
        self.sampler = Sampler(cfg.seed)
        self._next_id = 0
        self._inflight = None
        self.steps_ahead = 0           # decode steps queued before the step in front of them had been read
        self._tokenizer = None
        self._tokenizer_tried = False

    # ---- sizing ------------------------------------------------------------------------
    def _num_pages(self, model, dt, device) -> int:
        cfg = self.config
        if cfg.num_kvcache_slots and cfg.num_kvcache_slots > 0:
            return max(1, -(-int(cfg.num_kvcache_slots) // cfg.page_size))
        item = torch.empty((), dtype=dt).element_size()
        per_page = 0
        for req, layers in model.layout.groups:
            per_page = max(per_page, layers * 2 * req.num_kv_heads * cfg.page_size * req.head_dim * item)
        total_per_page = sum(layers * 2 * req.num_kv_heads * cfg.page_size * req.head_dim * item
                             for req, layers in model.layout.groups) or 1
        free, total = torch.cuda.mem_get_info(device)
        spec = model.spec
        workspace = cfg.max_num_batched_tokens * spec.hidden_size * item * 64 + (1 << 30)
        usable = int(total * cfg.gpu_memory_utilization) - (total - free) - workspace
        pages = usable // total_per_page
        cap = cfg.max_num_seqs_in_gpu * (-(-self.max_model_len // cfg.page_size))
        pages = min(pages, cap)
        if pages * cfg.page_size < min(self.max_model_len, 64):
            raise RuntimeError("not enough GPU memory left for a key/value cache")
        return int(pages)

    # ---- tokenizer (optional) ----------------------------------------------------------
    def _tok(self):
        if not self._tokenizer_tried:
            self._tokenizer_tried = True
            model = self.config.model
            if isinstance(model, str) and any(os.path.isfile(os.path.join(model, f))
                                              for f in ("tokenizer.json", "tokenizer.model")):
                from transformers import AutoTokenizer
                self._tokenizer = AutoTokenizer.from_pretrained(model, local_files_only=True)
        return self._tokenizer

    def _encode(self, prompt) -> list:
        if isinstance(prompt, str):
            tok = self._tok()
            if tok is None:
                raise ValueError("a string prompt needs a tokenizer in the model folder; pass token ids instead")
            return list(tok.encode(prompt))
        ids = [int(t) for t in prompt]
        vocab = self.runner.model.spec.vocab_size
        if not ids or min(ids) < 0 or max(ids) >= vocab:
            raise ValueError(f"prompt token ids must be a non-empty list within [0, {vocab})")
        return ids

    # ---- requests ----------------------------------------------------------------------
    def add_request(self, prompt, sampling_params: Optional[SamplingParams] = None) -> int:
        sp = sampling_params or SamplingParams()
        sp.validate_for_vocab(self.runner.model.spec.vocab_size)
        seq = Sequence(self._next_id, self._encode(prompt), sp)
        self.scheduler.add(seq)
        self._next_id += 1
        return seq.seq_id

    def abort_request(self, seq_id: int) -> bool:
        return self.scheduler.abort(seq_id)

    def is_finished(self) -> bool:
        return self.scheduler.is_finished() and self._inflight is None

    # ---- one step ------------------------------------------------------------------------
    # A step is queued on the device (forward pass, sampling, copies of the results to pinned
    # host memory) and read later.  With ``async_scheduling`` the next step of a batch that only
    # decodes is queued *before* this step's tokens are read: its input tokens are this step's
    # sampled ids, handed over on the device, so the GPU does not idle while the host reads
    # tokens, books them and prepares the next launch (the reference's asynchronous scheduling,
    # src/sparseengine/engine/llm_engine.py:1826-1957).  A request that turns out to have ended
    # (an end-of-sequence token, an abort) has then one token too many computed; it is dropped
    # when that step is read.

    def _launch(self, plan, feedback=None) -> "_InFlight":
        entries, reqs = [], []
        for it in plan.items:
            s = it.seq
            ahead = 1 if feedback is not None else 0          # tokens of this request still on their way
            toks = [0] if feedback is not None else s.slice(it.start, it.n_tokens)
            entries.append(StepEntry(s.seq_id, toks, [it.n_tokens - 1] if it.samples else []))
            if it.samples:
                reqs.append(SampleRequest(s.params, s.seq_id, len(s.output_ids) + ahead, s.prompt_ids, s.output_ids))
        logits = self.runner.step(entries, token_feedback=feedback)
        pending = None
        if reqs:
            from ..csrc import ops
            ops.error_enqueue(self.runner.device)
            pending = self.sampler.submit(logits, reqs)
        return _InFlight(plan, pending)

    def _may_run_ahead(self, cur: "_InFlight") -> bool:
        """Whether the step after ``cur`` can be queued before ``cur``'s tokens are known: every
        resident request decodes and is in ``cur``, none can end by length with the token on its
        way, nothing waits, nothing needs the tokens on the host, and the pages are there."""
        sch = self.scheduler
        if not self.config.async_scheduling or cur.pending is None or sch.waiting or cur.plan.preempted:
            return False
        items = cur.plan.items
        if len(items) != len(sch.running) or len(items) > self.config.max_decoding_seqs:
            return False
        for it, s in zip(items, sch.running):
            if it.seq is not s or it.n_tokens != 1 or not it.samples or not s.in_decode:
                return False
            p = s.params
            if p.has_penalties or p.benchmark_forced_token_ids is not None:
                return False
            if len(s.output_ids) + 2 > p.max_tokens or s.num_tokens + 2 > self.max_model_len:
                return False
        return self.runner.cache.can_reserve([(it.seq.seq_id, 1) for it in items])

    def step(self):
        cur = self._inflight
        self._inflight = None
        if cur is None:
            cur = self._launch(self.scheduler.schedule())
        nxt = None
        if self._may_run_ahead(cur):
            from .scheduler import Planned, StepPlan
            plan = StepPlan()
            plan.items = [Planned(it.seq, it.start + 1, 1, True) for it in cur.plan.items]
            nxt = self._launch(plan, feedback=cur.pending.tokens_device)
            self.steps_ahead += 1
        tokens, logprobs, tops = ([], None, None)
        if cur.pending is not None:
            from ..csrc import ops
            try:
                tokens, logprobs, tops = self.sampler.collect(cur.pending)
                ops.error_raise(self.runner.device)
            except BaseException:
                # This step's results cannot be used, and the step queued behind it was fed from
                # them.  Let that one finish (its pinned buffers are still in flight), then end
                # every request of this step: their cache no longer matches what the host knows of
                # them.  The engine stays usable for the requests that wait.
                if nxt is not None and nxt.pending is not None:
                    try:
                        self.sampler.collect(nxt.pending)
                    except Exception:
                        pass
                self.scheduler.fail(cur.plan, "error")
                raise
        live = sum(1 for it in cur.plan.items if it.seq.status == Status.RUNNING)
        decodes = min(cur.plan.num_decodes, live)
        prefill_tokens = cur.plan.num_tokens - cur.plan.num_decodes
        finished = self.scheduler.postprocess(cur.plan, tokens, logprobs, tops)
        self._inflight = nxt
        outs = [self._output(s) for s in finished]
        return outs, (prefill_tokens if prefill_tokens > 0 else -decodes)

    def _output(self, s: Sequence) -> dict:
        tok = self._tok() if self._tokenizer_tried or isinstance(self.config.model, str) else None
        text = tok.decode(s.output_ids, skip_special_tokens=True) if tok is not None else ""
        out = {"seq_id": s.seq_id, "text": text, "token_ids": list(s.output_ids), "finish_reason": s.finish_reason}
        if s.params.logprobs is not None and s.logprobs:
            out["logprobs"] = list(s.logprobs)
        if any(t is not None for t in s.top_logprobs):
            out["top_logprobs"] = list(s.top_logprobs)
        return out

    def generate(self, prompts: Seq, sampling_params=None, use_tqdm: bool = False) -> list:
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams per prompt (or a single one for all) is needed")
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]
        done: dict = {}
        bar = None
        if use_tqdm:
            from tqdm import tqdm
            bar = tqdm(total=len(ids), desc="generate", file=sys.stderr)
        import time
        interval = self.config.throughput_log_interval_s
        t_last, pre, dec = time.perf_counter(), 0, 0
        while not self.is_finished():
            outs, n = self.step()
            pre += max(n, 0)
            dec += max(-n, 0)
            for o in outs:
                done[o["seq_id"]] = o
                if bar is not None:
                    bar.update(1)
            now = time.perf_counter()
            if interval and now - t_last >= interval:
                print(f"[sparseengine_b200] prefill {pre / (now - t_last):.0f} tok/s, decode {dec / (now - t_last):.0f} tok/s, "
                      f"running {len(self.scheduler.running)}, waiting {len(self.scheduler.waiting)}, "
                      f"free pages {self.runner.cache.free_pages()}", file=sys.stderr, flush=True)
                t_last, pre, dec = now, 0, 0
        if bar is not None:
            bar.close()
        return [{k: v for k, v in done[i].items() if k != "seq_id"} for i in ids]

    def stats(self) -> dict:
        """Counters of the engine: steps, tokens, preemptions, cache occupancy, graph replays
        and, with ``enable_profiler``, milliseconds per part (CUDA events)."""
        c = self.runner.cache
        out = {"steps": self.runner.steps, "tokens": self.runner.tokens,
               "preemptions": self.scheduler.num_preemptions, "graph_replays": self.runner.graph_replays,
               "steps_ahead": self.steps_ahead,
               "waiting": len(self.scheduler.waiting), "running": len(self.scheduler.running),
               "free_rows": c.free_rows,
               "pages": [{"free": g.pool.free, "total": g.pool.num_pages, "taken": g.pool.taken_total,
                          "reused": g.pool.reused_total} for g in c.groups],
               "gpu_memory_allocated_bytes": torch.cuda.memory_allocated(self.runner.device)}
        prof = self.runner.model.profile
        if prof is not None:
            torch.cuda.synchronize(self.runner.device)
            out["part_ms"] = {k: round(sum(a.elapsed_time(b) for a, b in v), 3) for k, v in prof.items()}
        return out

    def exit(self) -> None:
        if self._inflight is not None and self._inflight.pending is not None:
            self.sampler.collect(self._inflight.pending)        # let what is queued finish
        self._inflight = None
        self.runner = None
        self.scheduler = None
        torch.cuda.empty_cache()
