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


def build_runner(model, *, dtype="bfloat16", page_size: int = 16, num_pages: int, max_rows: int,
                 max_seq_len: Optional[int] = None, device="cuda:0", random_weights: bool = False,
                 seed: int = 0, random_std: float = 0.02, decode_graphs: bool = True) -> ModelRunner:
    """``model`` is a folder (config.json + safetensors) or, with ``random_weights``, a
    folder or a config.json dictionary."""
    device = require_cuda(device)
    dt = resolve_dtype(dtype)
    typed, spec = load_model_spec(model)
    m = Model(spec, dt)
    with torch.cuda.device(device):
        if random_weights:
            init_random_(m, seed, device, std=random_std)
        else:
            load_weights(m, model, device)
        limit = int(max_seq_len) if max_seq_len else spec.max_position
        limit = min(limit, spec.max_position)
        cache = CacheManager(m.layout, page_size=page_size, num_pages=num_pages, max_rows=max_rows,
                             max_seq_len=limit, dtype=dt, device=device)
    return ModelRunner(m, cache, device, decode_graphs=decode_graphs)
