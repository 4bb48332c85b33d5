"""Python bindings of the exported kernel launchers (ctypes, raw device pointers).

Every launcher is ``extern "C" int se_<name>(..., cudaStream_t)``.  A binding checks
device, dtype and contiguity of each tensor, passes ``data_ptr()`` and the current
CUDA stream, and raises on a non-zero return.  There is no other implementation behind
these functions: without the compiled library they raise.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build as _build

_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_SIG = {"p": _P, "i": _I, "f": _F, "l": ctypes.c_longlong}

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}

_ERRORS = {-2: "a size this kernel does not support", -3: "an inconsistent argument"}

_fns: dict = {}

# Kernels launched through these bindings since the process started (a launcher that
# starts two kernels counts two).  Benchmarks read the difference around a timed region.
KERNELS_PER_CALL = {"se_attn_decode": 2, "se_router": 2}   # upper bounds per call
launch_count = 0
calls: dict = {}     # launcher name -> times called (tests check which kernels a path took)


def library():
    return _build.load()


# Sizes beyond which a kernel refuses (SE_ERR_UNSUPPORTED).  The parts check them when they are
# built, so that a model this library cannot run fails at construction with the limit named,
# not at its first step; the numbers restate the launchers' own (a GPU test compares them with
# what the compiled library reports through `limit`).
LIMITS = {
    "rmsnorm_max_width": 51200,             # a row is kept in shared memory in 32-bit
    "router_max_experts": 12800,            # four floats per expert in shared memory during selection
    "router_max_unaligned_width": 6400,     # widths that are no multiple of 4 keep 8 token rows in shared memory
    "moe_max_experts": 6079,                # the routing build's scans keep two ints per expert in shared memory
    "attention_max_head_dim": 256,          # in steps of 16
    "grid_dim_yz": 65535,                   # heads, KV heads and a step's entries map to grid dimensions y and z
}


def limit(name: str) -> int:
    """A size limit as the compiled library reports it."""
    f = getattr(library(), "se_" + name)
    f.restype = _I
    f.argtypes = []
    return int(f())


def _fn(name: str, sig: str):
    global launch_count
    launch_count += KERNELS_PER_CALL.get(name, 1)
    calls[name] = calls.get(name, 0) + 1
    f = _fns.get(name)
    if f is None:
        f = getattr(library(), name)
        f.restype = _I
        f.argtypes = [_SIG[c] for c in sig]
        _fns[name] = f
    return f


def _ptr(t: Optional[torch.Tensor], dtype=None, name: str = "tensor") -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check(code: int, what: str) -> None:
    if code == 0:
        return
    if code in _ERRORS:
        raise ValueError(f"{what}: {_ERRORS[code]}")
    raise RuntimeError(f"{what}: CUDA error {code}")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"activation dtype must be float32 or bfloat16, got {dtype}") from None


# ---- elementwise -------------------------------------------------------------------------

def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    tokens, hidden = out.shape
    _check(_fn("se_embed_gather", "pppiiiip")(
        _ptr(table, out.dtype, "table"), _ptr(ids, torch.int32, "ids"), _ptr(out), tokens, hidden,
        table.shape[0], dtype_code(out.dtype), _stream()), "embed_gather")
    return out


def rmsnorm(x, w, eps: float, out, residual=None, residual_out=None):
    """out = rmsnorm(x [+ residual]) * w; with a residual, residual_out = x + residual."""
    rows, hidden = x.shape
    if (residual is None) != (residual_out is None):
        raise ValueError("residual and residual_out go together")
    if w.shape != (hidden,):
        raise ValueError(f"norm weight shape {tuple(w.shape)} does not match width {hidden}")
    _check(_fn("se_rmsnorm", "pppppiifip")(
        _ptr(x, None, "x"), _ptr(residual, x.dtype, "residual"), _ptr(w, x.dtype, "w"), _ptr(out, x.dtype, "out"),
        _ptr(residual_out, x.dtype, "residual_out"), rows, hidden, float(eps), dtype_code(x.dtype), _stream()),
        "rmsnorm")
    return out


def gather_rows(src, idx, out):
    rows, width = out.shape
    _check(_fn("se_gather_rows", "pppiiip")(
        _ptr(src, out.dtype, "src"), _ptr(idx, torch.int32, "idx"), _ptr(out), rows, width,
        dtype_code(out.dtype), _stream()), "gather_rows")
    return out


def table_update(table, updates, n: int, num_pages: int):
    """Apply ``n`` (row, index, page) triples to a block table of a pool of ``num_pages`` pages."""
    _check(_fn("se_table_update", "piipiipp")(
        _ptr(table, torch.int32, "table"), table.shape[0], table.shape[1], _ptr(updates, torch.int32, "updates"), n,
        num_pages, _ptr(error_word(table.device)), _stream()), "table_update")


def table_update_dyn(table, updates, count, max_n: int, num_pages: int):
    _check(_fn("se_table_update_dyn", "piippiipp")(
        _ptr(table, torch.int32, "table"), table.shape[0], table.shape[1], _ptr(updates, torch.int32, "updates"),
        _ptr(count, torch.int32, "count"), max_n, num_pages, _ptr(error_word(table.device)), _stream()),
        "table_update_dyn")


# ---- attention ---------------------------------------------------------------------------

ROTARY_PAIRING = {"split_half": 0, "interleaved_to_split_half": 1, "interleaved": 3}


def qk_prep(qkv, q_w, k_w, inv_freq, positions, token_seq, seq_rows, table, cache, q_out, *, num_heads,
            num_kv_heads, head_dim, rotary_dim, eps, rope_scale, page_size, write_cache=True,
            pairing: str = "split_half", num_pages=None, step_inputs_settled: bool = False):
    """``num_pages``: the pool the block table's entries must lie in (default: the pages ``cache``
    holds); an entry outside it is not followed and shows in the error word.
    ``step_inputs_settled``: ``positions`` were complete before the kernel launched just before this
    call (the one that writes ``qkv``) began; the rotation angles are then computed while it runs."""
    tokens = qkv.shape[0]
    dt = qkv.dtype
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise ValueError("qkv width does not match the head counts")
    if pairing not in ROTARY_PAIRING:
        raise ValueError(f"rotary pairing {pairing!r} is not known; known: {sorted(ROTARY_PAIRING)}")
    inv_rms = None
    if q_w is not None and tokens > 64:      # many tokens: norm statistics once per token, not once per head
        inv_rms = torch.empty(tokens, 2, dtype=torch.float32, device=qkv.device)
    _check(_fn("se_qk_prep", "pppppppp" "ipp" "iiiii" "ff" "iip" "iip" "iip")(
        _ptr(qkv, None, "qkv"), _ptr(q_w, dt, "q_norm"), _ptr(k_w, dt, "k_norm"),
        _ptr(inv_freq, torch.float32, "inv_freq"), _ptr(positions, torch.int32, "positions"),
        _ptr(token_seq, torch.int32, "token_seq"), _ptr(seq_rows, torch.int32, "seq_rows"),
        _ptr(table, torch.int32, "table"), table.shape[1], _ptr(cache, dt, "cache"), _ptr(q_out, dt, "q_out"),
        tokens, num_heads, num_kv_heads, head_dim, rotary_dim, float(eps), float(rope_scale),
        page_size, int(write_cache), _ptr(inv_rms), ROTARY_PAIRING[pairing],
        cache.shape[0] if num_pages is None else int(num_pages), _ptr(error_word(qkv.device)),
        int(bool(step_inputs_settled)), dtype_code(dt), _stream()), "qk_prep")
    return q_out


def paged_attention_plain(q, cache, table, seq_rows, token_seq, positions, out, *, num_heads, num_kv_heads,
                          head_dim, page_size, scale, window=None, num_pages=None):
    tokens = q.shape[0]
    dt = q.dtype
    _check(_fn("se_paged_attention_plain", "pppipppp" "iiiii" "f" "iip" "ip")(
        _ptr(q, None, "q"), _ptr(cache, dt, "cache"), _ptr(table, torch.int32, "table"), table.shape[1],
        _ptr(seq_rows, torch.int32, "seq_rows"), _ptr(token_seq, torch.int32, "token_seq"),
        _ptr(positions, torch.int32, "positions"), _ptr(out, dt, "out"), tokens, num_heads, num_kv_heads,
        head_dim, page_size, float(scale), int(window or 0),
        cache.shape[0] if num_pages is None else int(num_pages), _ptr(error_word(q.device)),
        dtype_code(dt), _stream()), "paged_attention_plain")
    return out


# ---- feed-forward ------------------------------------------------------------------------

SCORE_FN = {"sigmoid": 0, "softmax": 1}


def router(x, gate, bias, ids, weights, *, top_k, score_fn="sigmoid", renormalize=True, routed_scale=1.0,
           logits_out=None):
    """32-bit router logits, scores, top-k and weights.  A token's logits are summed in one
    fixed order whatever the batch, so its experts do not depend on what shares its step."""
    tokens, hidden = x.shape
    experts = gate.shape[0]
    if gate.shape != (experts, hidden):
        raise ValueError("router weight shape does not match the activations")
    if logits_out is None:
        logits_out = torch.empty(tokens, experts, dtype=torch.float32, device=x.device)
    _check(_fn("se_router", "pppppp" "iiiii" "i" "f" "ip")(
        _ptr(x, None, "x"), _ptr(gate, torch.float32, "gate"), _ptr(bias, torch.float32, "bias"),
        _ptr(ids, torch.int32, "ids"), _ptr(weights, torch.float32, "weights"),
        _ptr(logits_out, torch.float32, "logits_out"), tokens, hidden, experts, top_k, SCORE_FN[score_fn],
        int(renormalize), float(routed_scale), dtype_code(x.dtype), _stream()), "router")
    return ids, weights


def router_select(logits, bias, ids, weights, *, top_k, score_fn="sigmoid", renormalize=True, routed_scale=1.0,
                  impl="auto"):
    """Selection alone from given 32-bit logits [tokens, experts], or from their parts
    [chunks, tokens, terms, experts], whose sum over chunks and terms (taken in that order inside the
    kernel) is the logit.  ``impl``: "auto", "block" (a block per token, any size and score function)
    or "warp" (a warp per token: sigmoid scores, up to 256 experts)."""
    if logits.dim() == 4:
        chunks, tokens, terms, experts = logits.shape
    else:
        (tokens, experts), chunks, terms = logits.shape, 1, 1
    _check(_fn("se_router_select", "pii" "ppp" "iiiii" "f" "ip")(
        _ptr(logits, torch.float32, "logits"), chunks, terms, _ptr(bias, torch.float32, "bias"),
        _ptr(ids, torch.int32, "ids"), _ptr(weights, torch.float32, "weights"), tokens, experts, top_k,
        SCORE_FN[score_fn], int(renormalize), float(routed_scale), {"auto": 0, "block": 1, "warp": 2}[impl], _stream()),
        "router_select")
    return ids, weights


def moe_plain_tile_rows() -> int:
    f = library().se_moe_plain_tile_rows
    f.restype = _I
    return int(f())


def moe_route_build(ids, experts: int, tile_rows: int, ws: dict, gather=None, stats=None):
    """ws: int32 tensors counts[E], rank[A], offsets[E+1], sorted[A], inv_pos[A],
    tile_expert[max_tiles], tile_row0[max_tiles], num_tiles[1].
    gather = (x [tokens, width], xs [A, width], top_k): also xs[p] = x[sorted[p] // top_k], the
    activation rows in expert order (in the same launch when there are few assignments).
    stats: optional int64[2] on the device; [0] += experts that got a row, [1] += 1.
    Returns whether the lists were complete before the last kernel of the build began (the
    gather of rows as a launch of its own): a grouped GEMM launched next may then read them
    while that kernel still runs (``lists_settled``)."""
    global launch_count
    assignments = ids.numel()
    x = xs = None
    top_k = row_bytes = 1
    if gather is not None:
        x, xs, top_k = gather
        if x.dtype != xs.dtype or x.shape[1] != xs.shape[1] or xs.shape[0] != assignments:
            raise ValueError("gather: xs must be [assignments, width] of x's dtype")
        row_bytes = x.shape[1] * x.element_size()
    small = bool(library().se_moe_route_is_small(assignments, experts))
    launch_count += (0 if small else 1) + (0 if small or gather is None else 1)
    _check(_fn("se_moe_route_gather", "piiii" "pppppppp" "ppi" "pp")(
        _ptr(ids, torch.int32, "ids"), assignments, experts, tile_rows, top_k,
        *[_ptr(ws[k], torch.int32, k) for k in ("counts", "rank", "offsets", "sorted", "inv_pos", "tile_expert",
                                                 "tile_row0", "num_tiles")],
        _ptr(x, None, "x"), _ptr(xs, None, "xs"), row_bytes, _ptr(stats, torch.int64, "stats"), _stream()),
        "moe_route_build")
    return not small and gather is not None


def moe_max_tiles(assignments: int, experts: int, tile_rows: int) -> int:
    return -(-assignments // tile_rows) + min(experts, assignments)


def moe_grouped_gemm_plain(mode: int, a, w, ws: dict, route_w, out, *, max_tiles, n_out, k_dim, top_k):
    dt = a.dtype
    _check(_fn("se_moe_grouped_gemm_plain", "i" "ppppppppp" "iiii" "ip")(
        mode, _ptr(a, None, "a"), _ptr(w, dt, "w"), _ptr(ws["sorted"]), _ptr(ws["offsets"]),
        _ptr(ws["tile_expert"]), _ptr(ws["tile_row0"]), _ptr(ws["num_tiles"]),
        _ptr(route_w, torch.float32, "route_w"), _ptr(out, dt, "out"), max_tiles, n_out, k_dim, top_k,
        dtype_code(dt), _stream()), "moe_grouped_gemm_plain")
    return out


def moe_combine(y, inv_pos, out, top_k: int):
    tokens, hidden = out.shape
    _check(_fn("se_moe_combine", "pppiiiip")(
        _ptr(y, out.dtype, "y"), _ptr(inv_pos, torch.int32, "inv_pos"), _ptr(out), tokens, hidden, top_k,
        dtype_code(out.dtype), _stream()), "moe_combine")
    return out


# ---- tensor-core GEMMs (bf16; csrc/gemm_tc.cu) ---------------------------------------------

_error_words = {}

# What a code in the error word says (csrc/common.cuh).
_WAIT_ROLES = "a tensor-core kernel timed out waiting on a barrier (role code {code}); its results are not valid"
_INDEX_CODES = {21: "the q/k preparation kernel", 22: "the plain attention kernel", 23: "the split-key decode attention kernel",
                24: "the prompt-portion attention kernel", 25: "the tcgen05 prompt-portion attention kernel",
                26: "the block-table update kernel"}


def error_text(code: int) -> str:
    if code in _INDEX_CODES:
        return (f"{_INDEX_CODES[code]} was given a block-table entry outside its page pool (code {code}); "
                "the access was skipped, the step's results are not valid")
    return _WAIT_ROLES.format(code=code)


def error_word(device) -> torch.Tensor:
    """The device word the kernels write when a bounded wait runs out or an index they were
    given points outside what they may touch (0 = all fine; the first code stays).  One per
    device, created on first use."""
    t = _error_words.get(device)
    if t is None:
        key = _device_key(device)
        t = _error_words.get(key)
        if t is None:
            t = torch.zeros(1, dtype=torch.int32, device=key)
            _error_words[key] = t
    return t


def _device_key(device) -> torch.device:
    key = torch.device(device)
    return torch.device(key.type, torch.cuda.current_device()) if key.index is None else key


def error_check(device) -> None:
    """Raise if a kernel reported a failure (reads one word from the device)."""
    t = _error_words.get(_device_key(device))
    if t is not None:
        code = int(t.item())
        if code:
            t.zero_()
            raise RuntimeError(error_text(code))


_error_host = {}


def error_enqueue(device) -> None:
    """Queue a copy of the error word to pinned host memory on the current stream: the step
    function calls this after a forward pass and reads the copy (:func:`error_raise`) once
    it has synchronised for its own results, so the check costs no synchronisation of its own."""
    key = _device_key(device)
    t = _error_words.get(key)
    if t is None:
        return
    h = _error_host.get(key)
    if h is None:
        h = torch.zeros(1, dtype=torch.int32).pin_memory()
        _error_host[key] = h
    h.copy_(t, non_blocking=True)


def error_raise(device) -> None:
    """Raise if the copy queued by :func:`error_enqueue` (and since completed) shows a failure."""
    key = _device_key(device)
    h = _error_host.get(key)
    if h is not None and int(h[0]):
        code = int(h[0])
        h.zero_()
        _error_words[key].zero_()
        raise RuntimeError(error_text(code))


def gemm_tc_supported(k_dim: int, n_out: int, nt: int = 16) -> bool:
    f = library().se_gemm_tc_supported
    f.restype = _I
    f.argtypes = [_I, _I, _I]
    return bool(f(k_dim, n_out, nt))


def moe_tile_rows_tc(assignments: int, experts: int) -> int:
    """Activation rows per tile for the tensor-core grouped GEMM: the power of two in [16, 256]
    that is at least 4/3 of the mean number of rows per expert.  A tile that holds fewer rows
    (an expert's last one) runs MMAs of its own rows only, so a large tile wastes no tensor
    work; what a tile size costs is shared memory per stage, what it saves is that an expert's
    weights cross from L2 to an SM once per tile.  Measured at M2 sizes over 256 experts
    (expert layer, ms, best first): 512 tokens 32 > 64 > 16; 1,024 and 1,536 tokens 64 > 32, 128;
    3,072 tokens 128 > 256 > 64; 4,096 tokens and more 256 > 128."""
    forced = os.environ.get("SE_MOE_TILE_ROWS")          # tuning aid
    if forced:
        return int(forced)
    want = -(-4 * assignments // (3 * max(experts, 1)))
    nt = 16
    while nt < want and nt < 256:
        nt *= 2
    return nt


def moe_grouped_gemm_tc(mode: int, a, w, ws: dict, route_w, out, *, experts, max_tiles, n_out, k_dim, nt,
                        lists_settled: bool = False):
    """``lists_settled``: the kernel launched just before this one does not write the lists in ``ws``
    (they were complete before it began).  The GEMM starts as a dependent of that kernel and then
    asks for its first weight tiles while it still runs; otherwise it waits for it first."""
    _check(_fn("se_moe_grouped_gemm_tc", "i" "pppppppppp" "iiiiiii" "p")(
        mode, _ptr(a, torch.bfloat16, "a"), _ptr(w, torch.bfloat16, "w"), _ptr(ws["sorted"]), _ptr(ws["offsets"]),
        _ptr(ws["tile_expert"]), _ptr(ws["tile_row0"]), _ptr(ws["num_tiles"]),
        _ptr(route_w, torch.float32, "route_w"), _ptr(out, torch.bfloat16, "out"), _ptr(error_word(a.device)),
        a.shape[0], experts, max_tiles, n_out, k_dim, nt, int(bool(lists_settled)), _stream()), "moe_grouped_gemm_tc")
    return out


PAIR_TILE_ROWS = 256      # activation rows per tile of the kernel that runs on pairs of SMs (csrc/gemm_tc_pair.cu)


def moe_grouped_gemm_pair_supported(k_dim: int, n_out: int) -> bool:
    f = library().se_moe_grouped_gemm_pair_supported
    f.restype = _I
    f.argtypes = [_I, _I]
    return bool(f(k_dim, n_out))


def moe_grouped_gemm_pair(mode: int, a, w, ws: dict, route_w, out, *, experts, max_tiles, n_out, k_dim):
    """The grouped expert GEMM on pairs of SMs (``tcgen05.mma.cta_group::2``, tiles of 256 x 256); the
    tile list in ``ws`` must have been built with ``PAIR_TILE_ROWS`` rows per tile."""
    _check(_fn("se_moe_grouped_gemm_pair", "i" "pppppppppp" "iiiii" "p")(
        mode, _ptr(a, torch.bfloat16, "a"), _ptr(w, torch.bfloat16, "w"), _ptr(ws["sorted"]), _ptr(ws["offsets"]),
        _ptr(ws["tile_expert"]), _ptr(ws["tile_row0"]), _ptr(ws["num_tiles"]),
        _ptr(route_w, torch.float32, "route_w"), _ptr(out, torch.bfloat16, "out"), _ptr(error_word(a.device)),
        a.shape[0], experts, max_tiles, n_out, k_dim, _stream()), "moe_grouped_gemm_pair")
    return out


def gemm_tc_dense(x, w, out, nt: int = 128):
    rows, k_dim = x.shape
    n_out = w.shape[0]
    _check(_fn("se_gemm_tc_dense", "pppp" "iiii" "p")(
        _ptr(x, torch.bfloat16, "x"), _ptr(w, torch.bfloat16, "w"), _ptr(out, torch.bfloat16, "out"),
        _ptr(error_word(x.device)), rows, n_out, k_dim, nt, _stream()), "gemm_tc_dense")
    return out


# ---- decode attention on tensor cores (bf16; csrc/attention_decode.cu) ----------------------

def attn_decode_supported(head_dim: int, num_heads: int, num_kv_heads: int) -> bool:
    f = library().se_attn_decode_supported
    f.restype = _I
    f.argtypes = [_I, _I, _I]
    return bool(f(head_dim, num_heads, num_kv_heads))


_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (asked once per device)."""
    key = torch.cuda.current_device() if device is None or torch.device(device).index is None else torch.device(device).index
    n = _sm_counts.get(key)
    if n is None:
        n = _sm_counts[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return n


def attn_decode_plan(tokens: int, num_heads: int, num_kv_heads: int, max_keys: int, sms: Optional[int] = None,
                     ctas_per_sm: int = 2):
    """How many key splits, and how many keys each.  CTAs = tokens x KV heads x splits run in
    waves of ``sms * ctas_per_sm`` (``sms``: the device's count unless given; two CTAs of the
    kernel fit an SM by shared memory); a CTA costs its 64-key tiles plus about three tiles of
    fixed work.  Pick the split count with the least waves x cost."""
    if sms is None:
        sms = sm_count()
    group = num_heads // num_kv_heads
    base = tokens * num_kv_heads * (-(-group // 16))
    slots = sms * ctas_per_sm
    tiles = -(-max_keys // 64)
    best = None
    for s in range(1, max(1, tiles // 2) + 1):
        per_tiles = -(-tiles // s)
        if s > 1 and -(-tiles // per_tiles) != s:
            continue                                  # the same split size as a smaller count
        waves = -(-base * s // slots)
        cost = waves * (per_tiles + 3)
        if best is None or cost < best[0]:
            best = (cost, s, per_tiles)
    _, splits, per_tiles = best
    return splits, per_tiles * 64


def attn_decode(q, cache, table, seq_rows, token_seq, positions, out, *, num_heads, num_kv_heads, head_dim, page_size,
                scale, window=None, max_keys: int, num_pages=None, step_inputs_settled: bool = False):
    """``step_inputs_settled``: ``table``, ``seq_rows``, ``token_seq`` and ``positions`` were complete
    before the kernel launched just before this call began (that kernel wrote ``q`` and the step's
    keys).  The attention kernel, launched as its dependent, then finds its place in the block table
    while it still runs; otherwise it waits for it first."""
    tokens = q.shape[0]
    splits, per = attn_decode_plan(tokens, num_heads, num_kv_heads, max_keys, sms=sm_count(q.device))
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty(tokens * num_heads * splits * head_dim, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(tokens * num_heads * splits * 2, dtype=torch.float32, device=q.device)
    _check(_fn("se_attn_decode", "pppipppppp" "iiiii" "f" "iii" "ip" "i" "p")(
        _ptr(q, torch.bfloat16, "q"), _ptr(cache, torch.bfloat16, "cache"), _ptr(table, torch.int32, "table"),
        table.shape[1], _ptr(seq_rows, torch.int32, "seq_rows"), _ptr(token_seq, torch.int32, "token_seq"),
        _ptr(positions, torch.int32, "positions"), _ptr(out, torch.bfloat16, "out"), _ptr(part_o), _ptr(part_ml),
        tokens, num_heads, num_kv_heads, head_dim, page_size, float(scale), int(window or 0), splits, per,
        cache.shape[0] if num_pages is None else int(num_pages), _ptr(error_word(q.device)),
        int(bool(step_inputs_settled)), _stream()),
        "attn_decode")
    return out


def attn_prefill(q, cache, table, seq_rows, cu_q, kv_len, out, *, entries, max_q_len, num_heads, num_kv_heads,
                 head_dim, page_size, scale, window=None, num_pages=None):
    _check(_fn("se_attn_prefill", "pppipppp" "iiiiii" "f" "i" "ip" "p")(
        _ptr(q, torch.bfloat16, "q"), _ptr(cache, torch.bfloat16, "cache"), _ptr(table, torch.int32, "table"),
        table.shape[1], _ptr(seq_rows, torch.int32, "seq_rows"), _ptr(cu_q, torch.int32, "cu_q"),
        _ptr(kv_len, torch.int32, "kv_len"), _ptr(out, torch.bfloat16, "out"), entries, max_q_len, num_heads,
        num_kv_heads, head_dim, page_size, float(scale), int(window or 0),
        cache.shape[0] if num_pages is None else int(num_pages), _ptr(error_word(q.device)), _stream()), "attn_prefill")
    return out


def attn_prefill_tc_supported(head_dim: int, num_heads: int, num_kv_heads: int) -> bool:
    f = library().se_attn_prefill_tc_supported
    f.restype = _I
    f.argtypes = [_I, _I, _I]
    return bool(f(head_dim, num_heads, num_kv_heads))


def attn_prefill_tc(q, cache, table, seq_rows, cu_q, kv_len, out, *, entries, max_q_len, num_heads, num_kv_heads,
                    head_dim, page_size, scale, window=None, num_pages=None):
    """Prompt-portion attention on tcgen05 (head size 128)."""
    _check(_fn("se_attn_prefill_tc", "pppippppp" "iiiiii" "f" "ii" "p")(
        _ptr(q, torch.bfloat16, "q"), _ptr(cache, torch.bfloat16, "cache"), _ptr(table, torch.int32, "table"),
        table.shape[1], _ptr(seq_rows, torch.int32, "seq_rows"), _ptr(cu_q, torch.int32, "cu_q"),
        _ptr(kv_len, torch.int32, "kv_len"), _ptr(out, torch.bfloat16, "out"), _ptr(error_word(q.device)),
        entries, max_q_len, num_heads, num_kv_heads, head_dim, page_size, float(scale), int(window or 0),
        cache.shape[0] if num_pages is None else int(num_pages), _stream()),
        "attn_prefill_tc")
    return out


# ---- dense projection for a handful of rows (bf16; csrc/gemv.cu) --------------------------------

def gemv_supported(rows: int, n_out: int, k_dim: int) -> bool:
    return 1 <= rows <= 16 and n_out >= 1 and k_dim >= 32 and k_dim % 32 == 0


def gemv(x, w, out):
    """out[rows <= 16, n] = x · wᵀ, weights streamed once through tensor-core fragments."""
    rows, k_dim = x.shape
    n_out = w.shape[0]
    _check(_fn("se_gemv", "pppiiip")(
        _ptr(x, torch.bfloat16, "x"), _ptr(w, torch.bfloat16, "w"), _ptr(out, torch.bfloat16, "out"), rows, n_out,
        k_dim, _stream()), "gemv")
    return out


# ---- read stream (csrc/read_stream.cu) ---------------------------------------------------------

def read_stream(t: torch.Tensor) -> None:
    """Read a contiguous tensor once with bulk asynchronous copies into shared memory, the way the
    weight-streaming GEMMs read HBM, and drop what arrives (a measuring aid: benchmarks time it)."""
    _check(_fn("se_read_stream", "plpp")(_ptr(t, None, "tensor"), t.numel() * t.element_size(),
                                         _ptr(error_word(t.device)), _stream()), "read_stream")
