"""Helpers shared by the replay tests: tiny model folders, traces in the four ways of
cutting, and the comparison with the plain implementation."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import torch

import plain_m2

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# name -> (config.json dict, seed, std, norm_std, bias_std, page size)
TINY = {
    "A": (plain_m2.TINY_A, 0, 0.02, 0.05, 0.0, 4),
    "B": (plain_m2.TINY_B, 1, 0.03, 0.0, 0.1, 8),
    "C": (plain_m2.TINY_C, 2, 0.05, 0.1, 0.05, 16),
    "D": (plain_m2.TINY_D, 3, 0.04, 0.05, 0.05, 16),
    "E": (plain_m2.TINY_E, 4, 0.04, 0.05, 0.1, 8),
}


def make_model_folder(folder: str, name: str, dtype: str = "float32") -> dict:
    """Write config.json + model.safetensors with the plain implementation's own random
    weights (so the engine's loader is tested against foreign tensors)."""
    from safetensors.torch import save_file
    cfg, seed, std, norm_std, bias_std, _ = TINY[name]
    tensors = plain_m2.random_tensors(cfg, seed, std, norm_std, bias_std)
    if dtype == "bfloat16":
        tensors = {k: (v if k.endswith(("gate.weight", "e_score_correction_bias")) else v.to(torch.bfloat16))
                   for k, v in tensors.items()}
    os.makedirs(folder, exist_ok=True)
    c = dict(cfg)
    c["torch_dtype"] = dtype
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(c, f)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    return tensors


def random_prompt(vocab: int, length: int, seed: int) -> list:
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()


# ---- traces: lists of steps {"step", "entries", "end"} ---------------------------------

def trace_whole(seqs: dict) -> list:
    steps = []
    for i, (sid, toks) in enumerate(seqs.items()):
        steps.append({"step": i, "entries": [{"id": sid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [sid]})
    return steps


def trace_tail_decode(seqs: dict, tail: int = 32) -> list:
    steps = []
    n = 0
    for sid, toks in seqs.items():
        head = max(1, len(toks) - tail)
        cuts = [(0, head)] + [(i, i + 1) for i in range(head, len(toks))]
        for a, b in cuts:
            steps.append({"step": n, "entries": [{"id": sid, "tokens": toks[a:b], "want": list(range(b - a))}],
                          "end": [sid] if b == len(toks) else []})
            n += 1
    return steps


def trace_chunks(seqs: dict, sizes=(7, 2, 5, 3, 2, 11, 4, 2, 9)) -> list:
    steps = []
    n = 0
    for sid, toks in seqs.items():
        a, k = 0, 0
        while a < len(toks):
            b = min(len(toks), a + sizes[k % len(sizes)])
            if len(toks) - b == 1:      # never leave a single last token: portions go down to two
                b = len(toks)
            steps.append({"step": n, "entries": [{"id": sid, "tokens": toks[a:b], "want": list(range(b - a))}],
                          "end": [sid] if b == len(toks) else []})
            n += 1
            a, k = b, k + 1
    return steps


def trace_mixed(seqs: dict, live: int = 4, chunk: int = 6, decode_tail: int = 5, seed: int = 0) -> list:
    """Up to ``live`` requests at a time: each is fed in chunks of ``chunk`` tokens until
    ``decode_tail`` tokens are left, which then go one per step; portions of some requests
    sit beside single tokens of others; a request is sometimes left out of a step; ended
    requests make room (and free pages) for waiting ones."""
    rng = np.random.RandomState(seed)
    waiting = list(seqs.items())
    active: dict = {}
    steps = []
    n = 0
    while waiting or active:
        while waiting and len(active) < live:
            sid, toks = waiting.pop(0)
            active[sid] = [toks, 0]
        entries, end = [], []
        ids = list(active)
        for sid in ids:
            toks, a = active[sid]
            if len(ids) > 1 and rng.rand() < 0.2:
                continue                      # left out of this step, goes on later
            left = len(toks) - a
            if left > decode_tail:
                b = a + min(chunk, left - decode_tail)
                if b - a == 1 and left - decode_tail == 1:
                    b = a + 1
            else:
                b = a + 1
            entries.append({"id": sid, "tokens": toks[a:b], "want": list(range(b - a))})
            active[sid][1] = b
            if b == len(toks):
                end.append(sid)
        for sid in end:
            del active[sid]
        if entries:
            steps.append({"step": n, "entries": entries, "end": end})
            n += 1
    return steps


def trace_random(seqs: dict, seed: int, live: int = 4) -> list:
    """A random schedule: requests start at random times (up to ``live`` at once), every step
    takes a random subset of them, each with one token, a few, or dozens (cut anywhere), and asks
    for the logits at all, some or none of them (the last token of a request is always asked
    for)."""
    rng = np.random.RandomState(seed)
    waiting = list(seqs.items())
    active: dict = {}
    steps = []
    n = 0
    while waiting or active:
        while waiting and len(active) < live and (not active or rng.rand() < 0.7):
            sid, toks = waiting.pop(0)
            active[sid] = [toks, 0]
        entries, end = [], []
        ids = list(active)
        for sid in ids:
            toks, a = active[sid]
            if len(ids) > 1 and rng.rand() < 0.25:
                continue
            kind = rng.rand()
            size = 1 if kind < 0.4 else int(rng.randint(2, 9)) if kind < 0.8 else int(rng.randint(9, 70))
            b = a + min(size, len(toks) - a)
            m = b - a
            pick = rng.rand()
            want = [] if pick < 0.15 else list(range(m)) if pick < 0.6 else sorted(
                set(int(x) for x in rng.randint(0, m, size=max(1, m // 2))))
            if b == len(toks) and (m - 1) not in want:
                want.append(m - 1)
            entries.append({"id": sid, "tokens": toks[a:b], "want": want})
            active[sid][1] = b
            if b == len(toks):
                end.append(sid)
        for sid in end:
            del active[sid]
        if entries:
            steps.append({"step": n, "entries": entries, "end": end})
            n += 1
    return steps


def max_live_tokens(steps, round_to: int = 64) -> int:
    """The --max-tokens a trace needs: the most tokens live requests hold at any time,
    each request's count rounded up to ``round_to``."""
    held: dict = {}
    worst = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-v // round_to) * round_to for v in held.values()))
        for sid in s["end"]:
            held.pop(sid, None)
    return worst


# ---- running a trace -------------------------------------------------------------------

def run_trace_cli(model_dir: str, dtype: str, steps: list, out_dir: str, max_tokens: int, extra=()) -> dict:
    """Run bin/trace_run as a subprocess; returns {(id, position): logits row}."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens), *extra]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for s in steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {s['step']}", f"expected 'done {s['step']}', got {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    return collect(steps, out_dir)


def collect(steps: list, out_dir: str, vocab: int | None = None) -> dict:
    out = {}
    pos: dict = {}
    for s in steps:
        wanted = [(e["id"], pos.get(e["id"], 0) + w) for e in s["entries"] for w in e["want"]]
        for e in s["entries"]:
            pos[e["id"]] = pos.get(e["id"], 0) + len(e["tokens"])
        for sid in s["end"]:
            pos.pop(sid, None)
        if not wanted:
            continue
        arr = np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4")
        arr = arr.reshape(len(wanted), -1)
        for key, row in zip(wanted, arr):
            out[key] = row
    return out


def run_trace_runner(runner, steps: list, capture: bool = False):
    """Run a trace in-process on a ModelRunner; returns {(id, position): logits row}.

    With ``capture`` it also returns the experts each routed feed-forward chose:
    ``{id: [visit][position] -> tuple of expert ids}``, one visit per routed feed-forward
    in the order the model runs them (a layer that runs twice counts twice)."""
    from sparseengine_b200.engine.runner import StepEntry
    out = {}
    pos: dict = {}
    routed: dict = {}
    parts = []
    if capture:
        runner.decode_graphs = False            # the capture hook copies to the host
        for entry in runner.model.spec.order:
            ff = runner.model.blocks[entry.layer].feed_forward
            if hasattr(ff, "route"):
                ff.capture = []
                parts.append(ff)
    for s in steps:
        entries = []
        for e in s["entries"]:
            if not runner.cache.has(e["id"]):
                runner.admit(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        logits = runner.step(entries)
        if capture:
            seen: dict = {}
            for visit, ff in enumerate(parts):          # a part visited twice appended twice, in order
                k = seen.get(id(ff), 0)
                seen[id(ff)] = k + 1
                ids = ff.capture[k].tolist()
                row = 0
                for e in s["entries"]:
                    store = routed.setdefault(e["id"], {}).setdefault(visit, {})
                    for j in range(len(e["tokens"])):
                        store[pos.get(e["id"], 0) + j] = tuple(ids[row])
                        row += 1
            for ff in parts:
                ff.capture = []
        wanted = [(e["id"], pos.get(e["id"], 0) + w) for e in s["entries"] for w in e["want"]]
        for e in s["entries"]:
            pos[e["id"]] = pos.get(e["id"], 0) + len(e["tokens"])
        if wanted:
            arr = logits.float().cpu().numpy()
            for key, row in zip(wanted, arr):
                out[key] = row
        for sid in s["end"]:
            runner.release(sid)
            pos.pop(sid, None)
    if capture:
        for ff in parts:
            ff.capture = None
        as_lists = {sid: [torch.tensor([v[p] for p in range(len(v))]) for _, v in sorted(visits.items())]
                    for sid, visits in routed.items()}
        return out, as_lists
    return out


def compare(got: dict, ref: dict, atol: float, rtol: float, what: str = ""):
    """ref: {id: [T, V] array}.  Reports the first wrong token."""
    worst = 0.0
    for (sid, p), row in sorted(got.items(), key=lambda kv: (str(kv[0][0]), kv[0][1])):
        want = ref[sid][p]
        err = np.abs(row - want)
        lim = atol + rtol * np.abs(want)
        if not (err <= lim).all():
            j = int(np.argmax(err - lim))
            raise AssertionError(f"{what}: request {sid!r} position {p}: logit {j} is {row[j]!r}, "
                                 f"plain gives {want[j]!r} (|diff| {err[j]:.3e} > {lim[j]:.3e})")
        worst = max(worst, float(err.max()))
    return worst


# bfloat16 against the plain implementation's bfloat16: both round at the same points, but sums
# inside a product run in another order, so values that land near the middle between two
# bfloat16 numbers round apart (half a unit in the last place, 2^-9 of the value), and the
# difference travels on through the layers.  The bound is stated in units of the logits' own
# size: a share of their root mean square over the compared rows, plus one unit in the last
# place (2^-7) of the logit itself.
BF16_SHARE_OF_RMS = 0.05
BF16_ULP = 2.0 ** -7


def compare_in_dtype(got: dict, ref: dict, dtype: str, what: str = "") -> float:
    """``compare`` with the bounds of the precision: 32-bit 1e-5 (the order of sums only);
    bfloat16 relative to the root mean square of the reference rows that are compared.
    Returns the worst difference in units of that root mean square."""
    rows = np.stack([ref[sid][p] for (sid, p) in got])
    rms = float(np.sqrt(np.mean(rows.astype(np.float64) ** 2)))
    if dtype == "float32":
        worst = compare(got, ref, 1e-5, 1e-5, what)
    else:
        worst = compare(got, ref, BF16_SHARE_OF_RMS * rms, BF16_ULP, what)
    print(f"[compare] {what}: logits rms {rms:.4f}, worst |diff| {worst:.3e} = {worst / max(rms, 1e-30):.4f} rms")
    return worst / max(rms, 1e-30)
