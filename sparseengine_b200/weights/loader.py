"""Load a model's parameters from ``*.safetensors`` by tensor name.

Every parameter lists the checkpoint tensors that fill it (packed q/k/v rows, one slice
per expert).  The whole folder is checked before anything is copied, and one error
lists every missing tensor, every unexpected tensor and every wrong shape.  Tensors go
to the engine's activation dtype, except parameters declared ``float32`` (router gate
and selection bias), which stay 32-bit whatever the engine dtype; integer tensors would
be kept as int32.  Names under the model's ignored prefixes, or that its
``ignored_rule`` accepts (multi-token-prediction modules), are skipped and counted.

Reference behaviour: src/sparseengine/utils/loader.py:674-904 (all shards, duplicate keys
are an error, strict validation), src/sparseengine/layers/linear.py:453-468 (qkv rows),
src/sparseengine/layers/packed_moe.py:189-261 (expert slices).
"""
from __future__ import annotations

import glob
import os
from dataclasses import dataclass, field

import torch
from safetensors import safe_open


class WeightLoadError(ValueError):
    """Raised once per load with everything that is wrong with the checkpoint."""

    def __init__(self, missing, unexpected, wrong_shape, other=()):
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)
        self.other = list(other)
        lines = ["checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: expected {tuple(e)}, found {tuple(f)}" for n, e, f in self.wrong_shape))
        for o in self.other:
            lines.append("  " + o)
        super().__init__("\n".join(lines))


@dataclass
class LoadReport:
    loaded: int = 0
    skipped: list = field(default_factory=list)


def _slice_shape(shape: tuple, index: tuple) -> tuple:
    out = []
    for i, dim in enumerate(shape):
        if i < len(index):
            ix = index[i]
            if isinstance(ix, int):
                continue
            out.append(ix[1])
        else:
            out.append(dim)
    return tuple(out)


def _dest(t: torch.Tensor, index: tuple) -> torch.Tensor:
    view = t
    dim = 0
    for ix in index:
        if isinstance(ix, int):
            view = view.select(dim, ix)
        else:
            view = view.narrow(dim, ix[0], ix[1])
            dim += 1
    return view


def checkpoint_files(model_dir: str) -> list[str]:
    files = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no *.safetensors file in {model_dir!r}")
    return files


def load_weights(model, model_dir: str, device) -> LoadReport:
    """Fill and bind every parameter of ``model`` from the folder's safetensors files."""
    params = model.params()
    expected: dict = {}     # checkpoint name -> (param, Source)
    for p in params:
        for src in p.sources:
            if src.name in expected:
                raise ValueError(f"checkpoint tensor {src.name!r} is claimed by two parameters")
            expected[src.name] = (p, src)

    files = checkpoint_files(model_dir)
    where: dict = {}
    shapes: dict = {}
    duplicates = []
    handles = []
    for path in files:
        try:
            f = safe_open(path, framework="pt", device="cpu")
        except Exception as e:      # a truncated or damaged file: say which one
            raise WeightLoadError([], [], [], [f"{path} cannot be read as safetensors ({type(e).__name__}: {e})"]) from e
        handles.append(f)
        for name in f.keys():
            if name in where:
                duplicates.append(f"tensor {name!r} appears in more than one file")
            where[name] = f
            shapes[name] = tuple(f.get_slice(name).get_shape())

    ignored = tuple(model.spec.ignored_prefixes)
    rule = getattr(model.spec, "ignored_rule", None)
    report = LoadReport()
    missing = sorted(n for n in expected if n not in where)
    unexpected = []
    for n in sorted(where):
        if n in expected:
            continue
        if (ignored and n.startswith(ignored)) or (rule is not None and rule(n)):
            report.skipped.append(n)
        else:
            unexpected.append(n)
    wrong = []
    for n, (p, src) in expected.items():
        if n in shapes:
            want = _slice_shape(tuple(p.spec.shape), src.index)
            if shapes[n] != want:
                wrong.append((n, want, shapes[n]))
    if missing or unexpected or wrong or duplicates:
        raise WeightLoadError(missing, unexpected, wrong, duplicates)

    for p in params:
        dtype = model.param_dtype(p.spec)
        p.tensor = torch.empty(tuple(p.spec.shape), dtype=dtype, device=device)
        for src in p.sources:
            t = where[src.name].get_tensor(src.name)
            if not (t.is_floating_point()):
                raise WeightLoadError([], [], [], [f"tensor {src.name!r} has dtype {t.dtype}, a floating type is needed"])
            _dest(p.tensor, src.index).copy_(t.to(device=device, dtype=dtype, non_blocking=False))
            report.loaded += 1
    model.bind(params)
    return report
