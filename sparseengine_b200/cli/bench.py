"""Command line in the reference's manner (benchmark/microbench.py:968-1071 of
CURRENTF/SparseEngine; wrapper scripts/benchmarks/bench_sparse_engine.py):

    python -m sparseengine_b200.cli.bench --model_path DIR --lengths 1024,4096 --batch_sizes 1,8 \
        --methods vanilla --output_len 64 --temperature 0 --top_p 1 \
        --hyper_params '{"max_num_batched_tokens": 8192}' --output_jsonl out.jsonl

Same option names and meanings where the option exists there: ``--lengths`` are prompt
lengths, ``--batch_sizes`` requests per case, ``--methods`` only ``vanilla`` (the dense
cache), ``--hyper_params`` the engine options as JSON or ``@file.json``.  The reference
feeds the constant prompt ``[100] * length``; ``--random_prompts`` draws seeded uniform
token ids instead (routing then spreads over the experts).  ``--generate`` prints the
generated token ids of each request instead of timing.  With ``--tiny_random`` the model
folder only needs a config.json; weights are random.
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def _ints(text: str) -> list:
    return [int(x) for x in text.split(",") if x.strip()]


def run_case(llm, length: int, batch: int, output_len: int, temperature: float, top_p: float, top_k: int,
             random_prompts: bool, seed: int, require_full: bool, warmup_steps: int, sync: bool) -> dict:
    import torch

    from sparseengine_b200 import SamplingParams
    vocab = llm.runner.model.spec.vocab_size
    g = torch.Generator().manual_seed(seed)
    prompts = [torch.randint(0, vocab, (length,), generator=g).tolist() if random_prompts else [100 % vocab] * length
               for _ in range(batch)]
    sp = SamplingParams(temperature=temperature, top_p=top_p, top_k=top_k, max_tokens=output_len, ignore_eos=True)
    for p in prompts:
        llm.add_request(p, sp)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    first_token_s = None
    prefill_tokens = 0
    prefill_s = decode_s = 0.0
    decode_tokens = 0
    full_steps = 0
    batch_sum = 0
    outputs = []
    while not llm.is_finished():
        t1 = time.perf_counter()
        outs, n = llm.step()
        if sync:
            torch.cuda.synchronize()
        dt = time.perf_counter() - t1
        outputs.extend(outs)
        if n > 0:
            prefill_tokens += n
            prefill_s += dt
        else:
            if first_token_s is None:
                first_token_s = t1 - t0
            if require_full and -n != batch:
                continue
            full_steps += 1
            if full_steps <= warmup_steps:
                continue
            decode_tokens += -n
            decode_s += dt
            batch_sum += -n
    torch.cuda.synchronize()
    total_s = time.perf_counter() - t0
    steps = max(full_steps - warmup_steps, 1)
    return {
        "method": "vanilla", "length": length, "batch_size": batch, "output_len": output_len,
        "first_token_s": first_token_s, "prefill_tok_s": prefill_tokens / prefill_s if prefill_s else None,
        "decode_tok_s": decode_tokens / decode_s if decode_s else None, "avg_decode_batch": batch_sum / steps,
        "total_s": total_s, "mem_gb": torch.cuda.max_memory_allocated() / 2**30,
        "preemptions": llm.scheduler.num_preemptions, "outputs": outputs,
    }


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Benchmark / generate with sparseengine_b200.")
    ap.add_argument("--model_path", required=True, help="folder with config.json (and safetensors)")
    ap.add_argument("--lengths", default="1024", help="prompt lengths, comma separated")
    ap.add_argument("--batch_sizes", default="1", help="requests per case, comma separated")
    ap.add_argument("--methods", default="vanilla", help="only 'vanilla' (the dense cache) exists here")
    ap.add_argument("--output_len", type=int, default=64, help="output tokens per request")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top_p", type=float, default=1.0)
    ap.add_argument("--top_k", type=int, default=0)
    ap.add_argument("--hyper_params", default="{}", help="engine options as JSON or @file.json")
    ap.add_argument("--output_jsonl", default=None)
    ap.add_argument("--max_model_len_override", type=int, default=None)
    ap.add_argument("--require_full_decode_batch", action="store_true",
                    help="count only decode steps in which every request of the case decodes")
    ap.add_argument("--decode_warmup_steps_after_full", type=int, default=0)
    ap.add_argument("--synchronize_step_timing", action="store_true")
    ap.add_argument("--tiny_random", action="store_true", help="random weights; the folder needs only config.json")
    ap.add_argument("--random_prompts", action="store_true", help="seeded uniform token ids instead of [100]*length")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--generate", action="store_true", help="print the generated token ids of every request")
    args = ap.parse_args(argv)

    methods = [m.strip() for m in args.methods.split(",") if m.strip()]
    if any(m != "vanilla" for m in methods):
        ap.error(f"only the 'vanilla' method exists in this engine, got {methods}")
    from sparseengine_b200 import LLM
    from sparseengine_b200.config.engine_config import Config
    lengths, batches = _ints(args.lengths), _ints(args.batch_sizes)
    Config.from_json(args.model_path, args.hyper_params)          # refuses unknown names early
    if args.hyper_params.startswith("@"):
        with open(args.hyper_params[1:]) as f:
            opts = json.load(f)
    else:
        opts = json.loads(args.hyper_params or "{}")
    if args.tiny_random:
        opts["tiny_random"] = True
    opts.setdefault("max_model_len", args.max_model_len_override or max(lengths) + args.output_len + 100)
    opts.setdefault("max_num_seqs_in_batch", max(max(batches), 32))
    llm = LLM(args.model_path, **opts)
    rows = []
    for length in lengths:
        for batch in batches:
            row = run_case(llm, length, batch, args.output_len, args.temperature, args.top_p, args.top_k,
                           args.random_prompts, args.seed, args.require_full_decode_batch,
                           args.decode_warmup_steps_after_full, args.synchronize_step_timing)
            outs = row.pop("outputs")
            rows.append(row)
            if args.generate:
                for o in sorted(outs, key=lambda o: o["seq_id"]):
                    print(json.dumps({"seq_id": o["seq_id"], "token_ids": o["token_ids"], "text": o["text"]}))
    if args.output_jsonl:
        with open(args.output_jsonl, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    hdr = ("method", "length", "batch", "first tok s", "prefill tok/s", "decode tok/s", "avg BS", "mem GB")
    print(" | ".join(hdr))
    for r in rows:
        def fmt(v, p=1):
            return "-" if v is None else f"{v:.{p}f}"
        print(" | ".join([r["method"], str(r["length"]), str(r["batch_size"]), fmt(r["first_token_s"], 3),
                          fmt(r["prefill_tok_s"]), fmt(r["decode_tok_s"]), fmt(r["avg_decode_batch"]), fmt(r["mem_gb"], 2)]))
    return 0


if __name__ == "__main__":
    sys.exit(main())
