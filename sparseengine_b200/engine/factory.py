"""Build a runner (model + weights + cache + step function) from a model folder."""
from __future__ import annotations

from typing import Optional

import torch

from .. import models  # noqa: F401  (registers the architectures)
from ..cache.manager import CacheManager
from ..config.registry import load_model_spec
from ..weights.loader import load_weights
from ..weights.random_init import init_random_
from .model import Model
from .runner import ModelRunner

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "fp32": torch.float32, "bf16": torch.bfloat16}


def resolve_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype must be float32 or bfloat16, got {dtype}")
        return dtype
    try:
        return DTYPES[str(dtype)]
    except KeyError:
        raise ValueError(f"dtype must be 'float32' or 'bfloat16', got {dtype!r}") from None


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("sparseengine_b200 runs on a CUDA device (sm_100a) only; no GPU is visible")
    return device


def build_runner(model, *, dtype="bfloat16", page_size: int = 16, num_pages, max_rows: int,
                 max_seq_len: Optional[int] = None, device="cuda:0", random_weights: bool = False,
                 seed: int = 0, random_std: float = 0.02, norm_std: float = 0.0, bias_std: float = 0.0,
                 decode_graphs: bool = True, state_slot_bytes: int = 0,
                 mlp_chunk_size: Optional[int] = None, kernel_tuning: Optional[dict] = None) -> ModelRunner:
    """The one place a model, its weights, its cache and its step function are put together
    (``LLM``, ``bin/trace_run``, the benchmarks and the tests all come through here).

    ``model`` is a folder (config.json + safetensors) or, with ``random_weights``, a folder or
    a config.json dictionary.  ``num_pages`` is a number, or a function of the built model
    (weights already on the device) that returns one: the entry point sizes the cache from the
    memory that the weights left.  ``norm_std`` / ``bias_std``: spread of random norm weights
    around 1 and of the random selection bias around 0.  ``kernel_tuning``: thresholds at which
    one kernel hands over to another (:data:`KERNEL_TUNING_KEYS`); they change speed, never
    results."""
    device = require_cuda(device)
    dt = resolve_dtype(dtype)
    typed, spec = load_model_spec(model)
    m = Model(spec, dt)
    with torch.cuda.device(device):
        if random_weights:
            init_random_(m, seed, device, std=random_std, norm_std=norm_std, bias_std=bias_std)
        else:
            load_weights(m, model, device)
        limit = int(max_seq_len) if max_seq_len else spec.max_position
        limit = min(limit, spec.max_position)
        pages = num_pages(m) if callable(num_pages) else num_pages
        cache = CacheManager(m.layout, page_size=page_size, num_pages=pages, max_rows=max_rows,
                             max_seq_len=limit, dtype=dt, device=device, reserved_state_bytes=state_slot_bytes)
    if mlp_chunk_size is not None:
        for b in m.blocks:
            for part in b.parts().values():
                if hasattr(part, "chunk_rows"):
                    part.chunk_rows = mlp_chunk_size
    apply_kernel_tuning(m, kernel_tuning or {})
    return ModelRunner(m, cache, device, decode_graphs=decode_graphs)


# option name -> (attribute of every part that has it, or of the module of dense projections)
KERNEL_TUNING_KEYS = {
    "attention_decode_kernel_max_tokens": "decode_kernel_max_tokens",   # larger steps take the prompt-portion attention kernel
    "attention_portion_min_tokens": "portion_min_tokens",               # ... and smaller ones whose longest entry has this many tokens
    "attention_portion_min_average": "portion_min_average",             # ... and this many tokens per entry on average
    "gemv_max_out_features": None,                                      # few-row projections wider than this take the library product
    "gemv_max_rows": None,                                              # ... and so do projections of more rows than this
    "router_tensor_core_min_tokens": "split_router_min_tokens",         # prompt steps from this size take router logits from tensor cores
    "moe_pair_min_rows": "pair_min_rows",                               # (token, slot) rows from which experts may run on pairs of SMs
    "moe_pair_min_rows_per_expert": "pair_min_rows_per_expert",         # ... if the experts that get rows have this many each
}


def check_kernel_tuning(tuning: dict) -> None:
    unknown = sorted(set(tuning) - set(KERNEL_TUNING_KEYS))
    if unknown:
        raise ValueError(f"unknown kernel_tuning key(s): {unknown}; known: {sorted(KERNEL_TUNING_KEYS)}")
    for k, v in tuning.items():
        if isinstance(v, bool) or not isinstance(v, int) or v < 0:
            raise ValueError(f"kernel_tuning[{k!r}] must be a non-negative integer, got {v!r}")


def apply_kernel_tuning(model: Model, tuning: dict) -> None:
    check_kernel_tuning(tuning)
    for key, value in tuning.items():
        attr = KERNEL_TUNING_KEYS[key]
        if attr is None:
            from ..parts import linear
            if key == "gemv_max_rows":
                linear.GEMV_MAX_ROWS = int(value)
            else:
                linear.GEMV_MAX_OUT = int(value)
            continue
        for b in model.blocks:
            for part in b.parts().values():
                if hasattr(part, attr):
                    setattr(part, attr, int(value))
