#!/usr/bin/env python3
"""Decode throughput of the engine at MiniMax M2 layer sizes, on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]

Prints ONE JSON line.  A "step" is one decode step of the whole batch (default: batch 8,
prompts of 2,048 tokens, context limit 4,096, bfloat16, random weights N(0, 0.02),
seed 2; layer sizes of MiniMax M2 at reduced depth).  ``value`` is decoded tokens per
second of the step function (device-timed, tokens stay on the device); ``e2e`` is the
same through ``LLM.add_request`` / ``LLM.step`` with host tokens in and out; ``prefill``
times one 2,048-token prompt; ``points`` are decode at batch 1 and 64, four prompts in one
step, and a long context (8 layers, one 131,072-token prompt in portions of 8,192 through
``LLM``, then 256 greedy steps); ``roofline`` is the bytes a decode step has to read (every
weight it uses once, the cache of the live requests) over its time, against the measured copy
bandwidth.  The caches the decode steps read were written by the step function (the requests'
2,048-token prompts are prefilled before timing); the experts a step touches are counted on
the timed steps themselves, by the routing build, on the device.

For --gpus N > 1 it prints one line that says so and exits with 2: the engine runs on
one GPU.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# MiniMax M2 layer sizes (the benchmark configuration), config.json keys.
M2_LAYER_SIZES = {
    "architectures": ["MiniMaxM2ForCausalLM"], "model_type": "minimax_m2",
    "hidden_size": 3072, "num_attention_heads": 48, "num_key_value_heads": 8, "head_dim": 128,
    "rotary_dim": 64, "rope_theta": 5000000.0, "rms_norm_eps": 1e-6,
    "num_local_experts": 256, "num_experts_per_tok": 8, "intermediate_size": 1536,
    "vocab_size": 200064, "max_position_embeddings": 4096, "tie_word_embeddings": False,
    "hidden_act": "silu", "qk_norm_type": "per_layer", "use_qk_norm": True, "scoring_func": "sigmoid",
    "use_routing_bias": True, "use_mtp": True, "shared_intermediate_size": 0, "torch_dtype": "bfloat16",
}
FULL_MODEL_LAYERS = 62
BENCH_LAYERS = 16
PROMPT_LEN = 2048
CONTEXT_LEN = 4096
PAGE_SIZE = 16
SEED = 2
LONG_LAYERS = 8
LONG_PROMPT = 131072
LONG_PORTION = 8192
LONG_STEPS = 256
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(FALLBACK_PEAKS)
    src = "fallback"
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if k in d and d[k]:
                    out[k] = float(d[k])
            src = "measured"
        except Exception:
            pass
    out["source"] = src
    return out


class ClockSampler:
    """nvidia-smi samples of the SM clock and throttle reasons while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, v in zip(self.NAMES, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_bytes(cfg: dict, layers: int):
    h, d = cfg["hidden_size"], cfg["head_dim"]
    hq, hkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    e, inter, v = cfg["num_local_experts"], cfg["intermediate_size"], cfg["vocab_size"]
    dense_layer = ((hq + 2 * hkv) * d * h + h * hq * d) * 2 + e * h * 4 + e * 4 + (2 * h + (hq + hkv) * d) * 2
    expert = 3 * inter * h * 2
    kv_token_layer = 2 * hkv * d * 2
    return {"dense_layer": dense_layer, "expert": expert, "lm_head": v * h * 2, "kv_token_layer": kv_token_layer,
            "weights_total": layers * (dense_layer + e * expert) + 2 * v * h * 2 + h * 2}


def prefill_flops(cfg: dict, layers: int, tokens: int) -> float:
    h, d = cfg["hidden_size"], cfg["head_dim"]
    hq, hkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    e, k, inter, v = cfg["num_local_experts"], cfg["num_experts_per_tok"], cfg["intermediate_size"], cfg["vocab_size"]
    per_token = 2 * h * (hq + 2 * hkv) * d + 2 * hq * d * h + 2 * h * e + k * 3 * 2 * h * inter
    attn = 4 * d * hq * tokens * (tokens + 1) / 2          # QK^T and PV, causal
    return layers * (tokens * per_token + attn) + 2 * h * v


def run_ours(args) -> dict:
    import torch

    from sparseengine_b200 import LLM, SamplingParams
    from sparseengine_b200.csrc import ops
    from sparseengine_b200.csrc import ops_sampling as sops
    from sparseengine_b200.engine.runner import StepEntry

    torch.cuda.set_device(0)
    cfg = dict(M2_LAYER_SIZES, num_hidden_layers=args.layers)
    pk = peaks()
    batch = args.batch
    max_rows = 64
    slots = max_rows * CONTEXT_LEN
    t0 = time.time()
    llm = LLM(cfg, tiny_random=True, tiny_random_seed=SEED, dtype="bfloat16", page_size=PAGE_SIZE,
              num_kvcache_slots=slots, max_model_len=CONTEXT_LEN, max_num_seqs_in_gpu=max_rows,
              max_num_seqs_in_batch=max_rows, max_decoding_seqs=max_rows, max_num_batched_tokens=8192,
              decode_reservation_tokens=0)
    torch.cuda.synchronize()
    setup_s = time.time() - t0
    runner = llm.runner
    vocab = cfg["vocab_size"]
    gen = torch.Generator().manual_seed(SEED)
    mb = model_bytes(cfg, args.layers)

    ffs = [b_.feed_forward for b_ in runner.model.blocks]

    def route_counters():
        """(experts that got a row, routing builds) summed over the layers, from the device."""
        torch.cuda.synchronize()
        got = [(f.route_stats + f.route_stats_large).tolist() if f.route_stats is not None else [0, 0] for f in ffs]
        return sum(g[0] for g in got), sum(g[1] for g in got)

    def fill(seq_ids, ctx):
        """Requests that hold ``ctx`` tokens: random prompts, prefilled through the step function
        (up to 8,192 tokens per step), so the decode steps read a cache the model wrote."""
        per_step = max(1, 8192 // ctx)
        for a in range(0, len(seq_ids), per_step):
            group = seq_ids[a:a + per_step]
            for s_ in group:
                runner.admit(s_)
            runner.step([StepEntry(s_, torch.randint(0, vocab, (ctx,), generator=gen).tolist(), []) for s_ in group])

    def decode_steps(seq_ids, n):
        toks = torch.randint(0, vocab, (n, len(seq_ids)), generator=gen).tolist()
        out = torch.empty(len(seq_ids), dtype=torch.int32, device="cuda")
        for i in range(n):
            logits = runner.step([StepEntry(s, [toks[i][j]], [0]) for j, s in enumerate(seq_ids)])
            sops.sample(logits, None, None, None, None, out)

    def timed_decode(b, ctx, warmup, steps, sample_clocks=False):
        ids = [f"b{b}_{i}" for i in range(b)]
        fill(ids, ctx)
        decode_steps(ids, warmup)
        torch.cuda.synchronize()
        sampler = ClockSampler()
        if sample_clocks:
            sampler.start()
        l0 = ops.launch_count
        used0, builds0 = route_counters()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        decode_steps(ids, steps)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        launches = ops.launch_count - l0
        clocks = sampler.stop() if sample_clocks else None
        # distinct experts per layer and step, counted by the routing builds of the timed steps
        used1, builds1 = route_counters()
        distinct = (used1 - used0) / max(builds1 - builds0, 1)
        for s in ids:
            runner.release(s)
        kv_ctx = ctx + warmup + steps // 2
        bytes_step = (args.layers * (mb["dense_layer"] + distinct * mb["expert"]) + mb["lm_head"]
                      + b * kv_ctx * args.layers * mb["kv_token_layer"])
        return {"ms": ms, "tok_s": b * 1000.0 / ms, "launches": launches, "clocks": clocks,
                "bytes": bytes_step, "distinct_experts_per_layer": distinct, "kv_ctx": kv_ctx}

    # ---- headline: decode at the default batch ------------------------------------------
    main = timed_decode(batch, PROMPT_LEN, args.warmup, args.steps, sample_clocks=True)
    if args.only_decode:
        return {"metric": "decode tokens/s", "value": round(main["tok_s"], 2), "ms_per_step": round(main["ms"], 4),
                "layers": args.layers, "global_batch": batch, "gpu_launches": main["launches"], "partial": True}
    points = {}
    for b in (1, 64):
        r = timed_decode(b, PROMPT_LEN, max(3, args.warmup), max(5, args.steps // 2))
        points[f"decode_b{b}"] = round(r["tok_s"], 2)
        points[f"decode_b{b}_hbm_frac"] = round(r["bytes"] / (r["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)

    # ---- prefill of one 2,048-token prompt ----------------------------------------------
    prompt = torch.randint(0, vocab, (PROMPT_LEN,), generator=gen).tolist()
    pre_ms, touched = [], []
    for i in range(7):                     # three to warm up, four timed: the fastest counts
        runner.admit(f"p{i}")
        used0, builds0 = route_counters()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        runner.step([StepEntry(f"p{i}", prompt, [PROMPT_LEN - 1])])
        e1.record()
        torch.cuda.synchronize()
        pre_ms.append(e0.elapsed_time(e1))
        used1, builds1 = route_counters()
        touched.append((used1 - used0) / max(builds1 - builds0, 1))
        runner.release(f"p{i}")
    pms = min(pre_ms[3:])
    flops = prefill_flops(cfg, args.layers, PROMPT_LEN)
    # hbm_frac: the bytes this prefill has to read (the weights of the experts it touches, counted
    # by the routing builds of the timed step, and the dense weights once; the prompt's K/V once)
    # over time and peak.  With random weights the deeper layers route most tokens to the same
    # experts, so the step touches far fewer than all experts; evenly routed it would be bound by
    # reading them all.
    per_layer = touched[pre_ms.index(pms)]
    pre_bytes = (args.layers * (mb["dense_layer"] + PROMPT_LEN * mb["kv_token_layer"] + per_layer * mb["expert"])
                 + mb["lm_head"])
    prefill = {"value": round(PROMPT_LEN * 1000.0 / pms, 1), "tokens": PROMPT_LEN, "ms": round(pms, 3),
               "frac": round(flops / (pms * 1e-3) / 1e12 / pk["bf16_tflops"], 4),
               "hbm_frac": round(pre_bytes / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
               "distinct_experts_per_layer": round(per_layer, 1)}
    prefill["binding_roof"] = "bf16 flops" if prefill["frac"] >= prefill["hbm_frac"] else "hbm bytes"

    # ---- an extra point: four such prompts in one step (8,192 tokens: towards compute-bound) ----
    prompts4 = [torch.randint(0, vocab, (PROMPT_LEN,), generator=gen).tolist() for _ in range(4)]
    ms4 = []
    for i in range(5):                     # two to warm up, three timed
        ids4 = [f"q{i}_{j}" for j in range(4)]
        for sid in ids4:
            runner.admit(sid)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        runner.step([StepEntry(sid, p, [PROMPT_LEN - 1]) for sid, p in zip(ids4, prompts4)])
        e1.record()
        torch.cuda.synchronize()
        ms4.append(e0.elapsed_time(e1))
        for sid in ids4:
            runner.release(sid)
    points["prefill_4x2048"] = round(4 * PROMPT_LEN * 1000.0 / min(ms4[2:]), 1)
    points["prefill_4x2048_frac"] = round(4 * flops / (min(ms4[2:]) * 1e-3) / 1e12 / pk["bf16_tflops"], 4)

    # ---- end to end through the public API -----------------------------------------------
    sp = SamplingParams(temperature=0.0, max_tokens=args.warmup + args.steps + 16, ignore_eos=True)
    for _ in range(batch):
        llm.add_request(torch.randint(0, vocab, (PROMPT_LEN,), generator=gen).tolist(), sp)
    while any(not s.in_decode for s in llm.scheduler.running) or llm.scheduler.waiting:
        llm.step()
    for _ in range(args.warmup):
        llm.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        _, n = llm.step()
        assert n == -batch, n
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    while not llm.is_finished():
        llm.step()
    h2d = 4 * (4 * (-(-batch // 4) * 4) + (-(-(batch + 1) // 4) * 4) + 4)      # packed int32 step metadata
    e2e = {"value": round(batch * args.steps / e2e_s, 2), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": 4 * batch}

    ops.error_check(llm.runner.device)       # a kernel that gave up on a wait would make every figure above void
    # a plain read of 4 GiB in this process: what a read-only stream reaches on this GPU, beside
    # the copy bandwidth (read + write) that the fraction is taken against
    buf = torch.empty(1 << 31, dtype=torch.bfloat16, device="cuda").fill_(1.0)
    best = 1e9
    for _ in range(6):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        buf.sum()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    read_stream = buf.numel() * 2 / (best * 1e-3) / 1e9
    # and the same bytes through bulk asynchronous copies into shared memory, as the expert GEMMs read
    best = 1e9
    for _ in range(6):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ops.read_stream(buf)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    tma_stream = buf.numel() * 2 / (best * 1e-3) / 1e9
    ops.error_check(llm.runner.device)
    del buf
    hbm = main["bytes"] / (main["ms"] * 1e-3) / 1e9
    if not args.no_long_context:
        llm.exit()
        del llm, runner, ffs
        torch.cuda.empty_cache()
        points.update(long_context(args, pk))
    return {
        "metric": f"decode tokens/s (MiniMax M2 layer sizes, batch {batch}, context 4096)",
        "value": round(main["tok_s"], 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main["ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform random token ids, random weights N(0,0.02) seed 2)",
        "impl": "ours",
        "config": {"model": "MiniMax-M2 layer sizes", "layers": args.layers, "layers_full_model": FULL_MODEL_LAYERS,
                   "hidden": 3072, "q_heads": 48, "kv_heads": 8, "head_dim": 128, "rotary_dim": 64,
                   "experts": 256, "top_k": 8, "expert_inter": 1536, "vocab": 200064, "global_batch": batch,
                   "seq_len": CONTEXT_LEN, "prompt_len": PROMPT_LEN, "page_size": PAGE_SIZE, "parallelism": "1gpu",
                   "l2": "working set per step >> L2 (no flush needed)", "cache": "prefilled by the step function",
                   "long_ctx": f"{LONG_LAYERS} layers, a {LONG_PROMPT}-token prompt in {LONG_PORTION}-token portions, "
                               f"{LONG_STEPS} greedy steps"},
        "clocks": main["clocks"], "e2e": e2e, "gpu_launches": main["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(hbm, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(hbm / pk["hbm_gbs"], 4), "peaks": pk["source"],
                     "read_stream_gbs": round(read_stream, 1), "bulk_copy_read_stream_gbs": round(tma_stream, 1),
                     "distinct_experts_per_layer": round(main["distinct_experts_per_layer"], 1)},
        "points": points, "setup_s": round(setup_s, 1),
    }


def long_context(args, pk) -> dict:
    """One 131,072-token prompt through ``LLM`` in portions of 8,192 (8 layers), then 256 greedy
    steps: what long block tables and the split of decode attention over the keys cost."""
    import torch

    from sparseengine_b200 import LLM, SamplingParams
    from sparseengine_b200.csrc import ops
    layers = args.long_layers
    cfg = dict(M2_LAYER_SIZES, num_hidden_layers=layers, max_position_embeddings=LONG_PROMPT + 1024)
    llm = LLM(cfg, tiny_random=True, tiny_random_seed=3, dtype="bfloat16", page_size=PAGE_SIZE,
              num_kvcache_slots=LONG_PROMPT + 1024, max_model_len=LONG_PROMPT + 1024, max_num_seqs_in_gpu=2,
              max_num_seqs_in_batch=2, max_decoding_seqs=2, max_num_batched_tokens=LONG_PORTION,
              engine_prefill_chunk_size=LONG_PORTION, decode_reservation_tokens=0)
    gen = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, cfg["vocab_size"], (LONG_PROMPT,), generator=gen).tolist()
    warm = 4
    llm.add_request(prompt, SamplingParams(temperature=0.0, max_tokens=warm + LONG_STEPS, ignore_eos=True))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    portions = 0
    while not llm.scheduler.running or not llm.scheduler.running[0].in_decode:
        llm.step()
        portions += 1
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    for _ in range(warm - 1):
        llm.step()
    torch.cuda.synchronize()
    ff = llm.runner.model.blocks[0].feed_forward
    t0 = time.perf_counter()
    steps = 0
    while not llm.is_finished():
        llm.step()
        steps += 1
    torch.cuda.synchronize()
    decode_ms = (time.perf_counter() - t0) * 1e3 / max(steps, 1)
    ops.error_check(llm.runner.device)
    mb = model_bytes(cfg, layers)
    flops = prefill_flops(cfg, layers, LONG_PROMPT)
    kv_bytes = (LONG_PROMPT + warm + LONG_STEPS // 2) * layers * mb["kv_token_layer"]
    read = layers * (mb["dense_layer"] + cfg["num_experts_per_tok"] * mb["expert"]) + mb["lm_head"] + kv_bytes
    llm.exit()
    sustained = pk.get("bf16_tflops_sustained", pk["bf16_tflops"])
    return {"long_ctx_layers": layers, "long_ctx_prompt": LONG_PROMPT, "long_ctx_portions": portions,
            "long_ctx_prefill_tok_s": round(LONG_PROMPT / prefill_s, 1), "long_ctx_prefill_s": round(prefill_s, 3),
            "long_ctx_prefill_frac": round(flops / prefill_s / 1e12 / pk["bf16_tflops"], 4),
            "long_ctx_prefill_frac_sustained": round(flops / prefill_s / 1e12 / sustained, 4),
            "long_ctx_decode_steps": steps, "long_ctx_decode_ms": round(decode_ms, 4),
            "long_ctx_decode_tok_s": round(1000.0 / decode_ms, 2),
            "long_ctx_decode_hbm_frac": round(read / (decode_ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)}


def run_reference(args) -> dict:
    """The unmodified reference from ``baseline/_ref`` through its own public API
    (``sparseengine.LLM(folder, tiny_random=True, ...).generate``): the same layer sizes, batch
    and prompt length.  Whatever stops it (it checks its kernel packages when the engine starts,
    src/sparseengine/kernels/external/required.py:39, and has only an FP8 path for MiniMax M2,
    src/sparseengine/models/spec.py:161-173) is caught and reported as ``unavailable``; on an
    image where it starts, the same code gives its number."""
    import tempfile
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "sparseengine")):
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed (pip install --no-index --no-deps "
                                                    "--target baseline/_ref <reference checkout>)"}
    sys.path.insert(0, ref)
    folder = None
    try:
        import torch
        from sparseengine import LLM, SamplingParams            # the reference's own entry point
        folder = tempfile.mkdtemp(prefix="ref_m2_")
        # the reference reads MiniMax M2 only with its published quantization (FP8 block scales)
        cfg = dict(M2_LAYER_SIZES, num_hidden_layers=FULL_MODEL_LAYERS, max_position_embeddings=204800,
                   num_mtp_modules=3, mtp_transformer_layers=1,
                   quantization_config={"quant_method": "fp8", "fmt": "float8_e4m3fn", "activation_scheme": "dynamic",
                                        "weight_block_size": [128, 128],
                                        "modules_to_not_convert": ["gate", "e_score_correction_bias", "lm_head"]})
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(cfg, f)
        tiny = os.path.join(folder, "tiny.json")
        with open(tiny, "w") as f:
            json.dump({"num_hidden_layers": args.layers, "hidden_size": cfg["hidden_size"],
                       "intermediate_size": cfg["intermediate_size"]}, f)
        from tokenizers import Tokenizer
        from tokenizers.models import WordLevel
        tok = Tokenizer(WordLevel({f"t{i}": i for i in range(cfg["vocab_size"])}, unk_token="t0"))
        tok.save(os.path.join(folder, "tokenizer.json"))
        with open(os.path.join(folder, "tokenizer_config.json"), "w") as f:
            json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "t1", "unk_token": "t0",
                       "pad_token": "t0"}, f)
        llm = LLM(folder, tiny_random=True, tiny_random_config=tiny, max_model_len=CONTEXT_LEN,
                  max_num_batched_tokens=8192, max_num_seqs_in_batch=args.batch)
        gen = torch.Generator().manual_seed(SEED)
        prompts = [torch.randint(0, cfg["vocab_size"], (PROMPT_LEN,), generator=gen).tolist() for _ in range(args.batch)]

        def timed(n):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True))
            torch.cuda.synchronize()
            return time.perf_counter() - t0
        timed(max(args.warmup, 3))
        # decode time = a run of warmup + steps tokens minus a run of warmup tokens (the prefill cancels)
        short, long_ = timed(args.warmup), timed(args.warmup + args.steps)
        ms = (long_ - short) * 1e3 / args.steps
        return {"metric": f"decode tokens/s (MiniMax M2 layer sizes, batch {args.batch}, context 4096)",
                "value": round(args.batch * 1000.0 / ms, 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "impl": "reference",
                "dtype": "fp8 weights (the reference's only MiniMax M2 path)", "data": "synthetic, tiny_random weights",
                "e2e": {"value": round(args.batch * 1000.0 / ms, 2), "unit": "tokens/s"}}
    except BaseException as exc:             # the reference's refusal, in its own words
        text = " ".join(str(exc).split())
        return {"impl": "reference", "unavailable": f"the unmodified reference did not run here: {type(exc).__name__}: {text[:600]}"}
    finally:
        if folder is not None:
            import shutil
            shutil.rmtree(folder, ignore_errors=True)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--layers", type=int, default=BENCH_LAYERS)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-long-context", action="store_true", help="leave out the 131,072-token point")
    ap.add_argument("--long-layers", type=int, default=LONG_LAYERS)
    ap.add_argument("--only-decode", action="store_true",
                    help="time the headline decode only (no points, prefill or end-to-end run): for profiling")
    args = ap.parse_args()
    if args.impl == "reference":
        # the reference logs to standard output; this arm's one line must be alone there
        sys.stdout.flush()
        keep = os.dup(1)
        os.dup2(2, 1)
        try:
            rec = run_reference(args)
        finally:
            sys.stdout.flush()
            os.dup2(keep, 1)
            os.close(keep)
        print(json.dumps(rec))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
