"""Trace replay on top of the engine's own step function (used by ``bin/trace_run``)."""
from __future__ import annotations

import json
import os

import torch

from .engine.factory import build_runner
from .engine.runner import StepEntry


def replay(model_dir: str, dtype: str, out_dir: str, max_tokens: int, *, page_size: int = 16,
           max_requests: int = 8, device="cuda:0", lines=(), log=None) -> int:
    if 64 % page_size:
        raise ValueError("page size must divide 64 (live requests are counted in multiples of 64 tokens)")
    from .csrc import ops
    ops.library()          # compile (first call) and load before anything else; fails loudly
    os.makedirs(out_dir, exist_ok=True)
    num_pages = max(1, -(-max_tokens // page_size))
    runner = build_runner(model_dir, dtype=dtype, page_size=page_size, num_pages=num_pages,
                          max_rows=max_requests, device=device)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        entries = []
        for e in rec.get("entries", []):
            if not runner.cache.has(e["id"]):
                runner.admit(e["id"])
            entries.append(StepEntry(e["id"], list(e["tokens"]), list(e.get("want", []))))
        logits = runner.step(entries)
        if logits is not None and logits.shape[0] > 0:
            ops.error_enqueue(runner.device)
            arr = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
            ops.error_raise(runner.device)
            arr.tofile(os.path.join(out_dir, f"{rec['step']}.f32"))
        else:
            ops.error_enqueue(runner.device)
            torch.cuda.synchronize(runner.device)
            ops.error_raise(runner.device)
        for seq_id in rec.get("end", []):
            if runner.cache.has(seq_id):
                runner.release(seq_id)
        if log is not None:
            print(f"done {rec['step']}", file=log, flush=True)
    return 0
