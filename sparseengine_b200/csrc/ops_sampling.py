"""Bindings of the sampling kernels (csrc/sampling.cu)."""
from __future__ import annotations

import torch

from .ops import _check, _fn, _ptr, _stream, dtype_code


def sample(logits, temperature, top_k, top_p, seeds, out, logprob=None, impl: int = 0):
    rows, vocab = logits.shape
    if temperature is None and logprob is None and vocab >= 16384:
        # greedy over a large vocabulary: two stages, many blocks per row
        pval = torch.empty(rows * 64, dtype=torch.float32, device=logits.device)
        pidx = torch.empty(rows * 64, dtype=torch.int32, device=logits.device)
        _check(_fn("se_argmax", "pppp" "iii" "p")(
            _ptr(logits, None, "logits"), _ptr(out, torch.int32, "out"), _ptr(pval), _ptr(pidx), rows, vocab,
            dtype_code(logits.dtype), _stream()), "argmax")
        return out
    if (impl == 0 and temperature is not None and top_k is None and top_p is None and vocab >= 16384
            and rows <= 256):
        # no cuts, a large vocabulary, few rows: many blocks per row
        f32 = dict(dtype=torch.float32, device=logits.device)
        i32 = dict(dtype=torch.int32, device=logits.device)
        ws = [torch.empty(rows * 64, **f32), torch.empty(rows * 64, **i32), torch.empty(rows * 64, **f32),
              torch.empty(rows * 64, **f32), torch.empty(rows * 64, **i32)]
        _check(_fn("se_sample_plain", "ppppp" "ppppp" "iii" "p")(
            _ptr(logits, None, "logits"), _ptr(temperature, torch.float32, "temperature"),
            _ptr(seeds, torch.int64, "seeds"), _ptr(out, torch.int32, "out"), _ptr(logprob, torch.float32, "logprob"),
            *[_ptr(w) for w in ws], rows, vocab, dtype_code(logits.dtype), _stream()), "sample_plain")
        return out
    spill = None
    if impl == 0 and temperature is not None and (top_k is not None or top_p is not None):
        # room for a row's list of candidates when it does not fit into shared memory: three
        # arrays of up to a quarter of the row each (a longer list takes the whole-row form)
        spill = torch.empty(rows * 3 * (-(-vocab // 4)), dtype=torch.float32, device=logits.device)
    _check(_fn("se_sample", "pppppppp" "iiii" "p")(
        _ptr(logits, None, "logits"), _ptr(temperature, torch.float32, "temperature"),
        _ptr(top_k, torch.int32, "top_k"), _ptr(top_p, torch.float32, "top_p"), _ptr(seeds, torch.int64, "seeds"),
        _ptr(out, torch.int32, "out"), _ptr(logprob, torch.float32, "logprob"), _ptr(spill), rows, vocab,
        dtype_code(logits.dtype), impl, _stream()), "sample")
    return out


def apply_penalties(logits, pairs, n, repetition, presence):
    rows, vocab = logits.shape
    _check(_fn("se_apply_penalties", "ppiippp")(
        _ptr(logits, torch.float32, "logits"), _ptr(pairs, torch.int32, "pairs"), n, vocab,
        _ptr(repetition, torch.float32, "repetition"), _ptr(presence, torch.float32, "presence"), _stream()),
        "apply_penalties")


def to_float(src, dst):
    _check(_fn("se_to_float", "pplip")(
        _ptr(src, None, "src"), _ptr(dst, torch.float32, "dst"), src.numel(), dtype_code(src.dtype), _stream()),
        "to_float")
    return dst


def top_logprobs(logits, rows, ids, values):
    """The ``ids.shape[1]`` most likely tokens of the listed rows with their log-probabilities
    (32-bit log-softmax), most likely first."""
    count, n = ids.shape
    _check(_fn("se_top_logprobs", "pppp" "iiii" "p")(
        _ptr(logits, None, "logits"), _ptr(rows, torch.int32, "rows"), _ptr(ids, torch.int32, "ids"),
        _ptr(values, torch.float32, "values"), count, logits.shape[1], n, dtype_code(logits.dtype), _stream()),
        "top_logprobs")
    return ids, values
