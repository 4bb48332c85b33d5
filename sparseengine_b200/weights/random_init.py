"""Random weights: write a model folder (config.json + model.safetensors) from a
configuration and a seed, or fill a built model in place on its device.

Each checkpoint tensor draws from a generator seeded by (seed, tensor name), so a
folder can be produced tensor by tensor and any subset reproduces.  Distributions:
matrices N(0, std); norm weights 1 + N(0, norm_std); selection bias N(0, bias_std).
The reference's counterpart is its tiny-random debug mode
(src/sparseengine/debug/tiny_random.py:255-292: every float parameter N(0, 0.02) from one
seeded generator).
"""
from __future__ import annotations

import hashlib
import json
import os

import torch
from safetensors.torch import save_file

from ..config.registry import load_model_spec
from ..engine.model import Model
from .loader import _dest, _slice_shape

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _name_seed(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little") & (2**63 - 1)


def _draw(shape, init: str, seed: int, name: str, device, std, norm_std, bias_std) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_name_seed(seed, name))
    x = torch.randn(tuple(shape), generator=g, device=device, dtype=torch.float32)
    if init == "norm":
        return 1.0 + x * norm_std
    if init == "bias":
        return x * bias_std
    return x * std


def write_random_model(folder: str, config: dict, seed: int, *, std: float = 0.02, norm_std: float = 0.0,
                       bias_std: float = 0.0, dtype: str = "float32") -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a config.json
    dictionary of a registered architecture).  ``dtype`` is the stored dtype; tensors the
    model keeps in 32-bit (router gate, selection bias) are stored in 32-bit."""
    if dtype not in _DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}")
    typed, spec = load_model_spec(config)
    model = Model(spec, _DTYPES[dtype])
    tensors = {}
    for p in model.params():
        store = torch.float32 if p.spec.dtype == "float32" else _DTYPES[dtype]
        for src in p.sources:
            shape = _slice_shape(tuple(p.spec.shape), src.index)
            tensors[src.name] = _draw(shape, p.spec.init, seed, src.name, "cpu", std, norm_std, bias_std).to(store)
    os.makedirs(folder, exist_ok=True)
    cfg = dict(config)
    cfg["torch_dtype"] = dtype
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    return folder


def init_random_(model: Model, seed: int, device, *, std: float = 0.02, norm_std: float = 0.0,
                 bias_std: float = 0.0, per_source: bool = False, chunk_elems: int = 1 << 27) -> None:
    """Fill every parameter of ``model`` with seeded random values directly on ``device``
    and bind them.  With ``per_source=True`` each checkpoint tensor is drawn on its own
    (same values as :func:`write_random_model` when ``device`` is the CPU); otherwise
    each packed parameter is drawn in large chunks, which is what a benchmark with
    ~100 GB of weights wants."""
    params = model.params()
    for p in params:
        dtype = model.param_dtype(p.spec)
        p.tensor = torch.empty(tuple(p.spec.shape), dtype=dtype, device=device)
        if per_source:
            for src in p.sources:
                shape = _slice_shape(tuple(p.spec.shape), src.index)
                _dest(p.tensor, src.index).copy_(
                    _draw(shape, p.spec.init, seed, src.name, device, std, norm_std, bias_std))
            continue
        flat = p.tensor.view(-1)
        g = torch.Generator(device=device)
        g.manual_seed(_name_seed(seed, p.qualified))
        for start in range(0, flat.numel(), chunk_elems):
            n = min(chunk_elems, flat.numel() - start)
            x = torch.randn(n, generator=g, device=device, dtype=torch.float32)
            if p.spec.init == "norm":
                x = 1.0 + x * norm_std
            elif p.spec.init == "bias":
                x = x * bias_std
            else:
                x = x * std
            flat[start:start + n].copy_(x)
    model.bind(params)
