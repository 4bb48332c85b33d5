"""Engine options: one flat record with the reference's names where the concept
survives (src/sparseengine/configs/runtime.py:51-110, src/sparseengine/configs/scheduling.py:15-93),
shared by ``LLM(...)``, JSON (``--hyper_params``) and the engine's own parts.  Unknown
names are refused (src/sparseengine/engine/llm_engine.py:232-239).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, fields
from typing import Optional


@dataclass
class Config:
    model: str                                     # folder with config.json (+ safetensors)
    # scheduling (reference names)
    max_num_batched_tokens: int = 8192             # token budget of one step
    max_num_seqs_in_batch: int = 32                # most prompt portions in one step
    max_model_len: Optional[int] = None            # default: the model's context length
    max_decoding_seqs: Optional[int] = None        # default: max_num_seqs_in_batch
    max_num_seqs_in_gpu: Optional[int] = None      # rows; default max(3*batch, decoding)
    engine_prefill_chunk_size: Optional[int] = None  # default: the token budget
    decode_reservation_tokens: int = 1024          # future tokens promised to each resident request
    prefill_schedule_policy: str = "auto"          # "auto" | "all_chunked"
    gpu_memory_utilization: float = 0.9
    num_kvcache_slots: int = -1                    # tokens of cache; -1 = from memory
    tensor_parallel_size: int = 1
    expert_parallel_size: int = 1
    data_parallel_size: int = 1
    sparse_method: str = ""                        # "" or "vanilla": the dense cache
    mlp_chunk_size: int = 16384                    # most rows the feed-forward takes at once
    decode_graph: bool = True                      # replay decode steps as CUDA graphs
    async_scheduling: bool = True                  # queue the next decode step before the host has read this one's tokens
    enable_profiler: bool = False                  # CUDA-event timing of every part (forces launch-by-launch steps)
    validate_runtime_invariants: bool = False      # host-side checks of every step's index tensors
    throughput_log_interval_s: float = 10.0        # generate() logs tokens/s this often (0 = never)
    tiny_random: bool = False                      # random weights instead of a checkpoint
    tiny_random_config: Optional[str] = None       # JSON file of size overrides for the model's config.json
    tiny_random_seed: int = 0
    tiny_random_std: float = 0.02                  # random matrices N(0, std)
    tiny_random_norm_std: float = 0.0              # random norm weights 1 + N(0, std)
    tiny_random_bias_std: float = 0.0              # random router selection bias N(0, std)
    eos: int = -1
    eos_token_ids: tuple = field(default_factory=tuple)
    # this engine's own
    dtype: str = "bfloat16"                        # "bfloat16" | "float32"
    page_size: int = 16
    seed: int = 0                                  # sampler seed
    device: str = "cuda:0"
    state_slot_bytes: int = 0                      # reserved per-request state for sparse methods (unused)
    kernel_tuning: dict = field(default_factory=dict)   # thresholds between kernels (engine/factory.py: KERNEL_TUNING_KEYS)

    def __post_init__(self):
        if self.sparse_method not in ("", "vanilla"):
            raise ValueError(f"sparse_method {self.sparse_method!r} is not supported (only the dense 'vanilla' cache)")
        for name in ("tensor_parallel_size", "expert_parallel_size", "data_parallel_size"):
            if getattr(self, name) != 1:
                raise ValueError(f"{name} must be 1 (one GPU)")
        if self.prefill_schedule_policy not in ("auto", "all_chunked"):
            raise ValueError("prefill_schedule_policy must be 'auto' or 'all_chunked'")
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError("dtype must be 'bfloat16' or 'float32'")
        if self.max_num_batched_tokens <= 0 or self.max_num_seqs_in_batch <= 0 or self.page_size <= 0:
            raise ValueError("max_num_batched_tokens, max_num_seqs_in_batch and page_size must be positive")
        if not 0.0 < self.gpu_memory_utilization <= 1.0:
            raise ValueError("gpu_memory_utilization must be in (0, 1]")
        if self.max_decoding_seqs is None:
            self.max_decoding_seqs = self.max_num_seqs_in_batch
        if self.max_num_seqs_in_gpu is None:
            self.max_num_seqs_in_gpu = max(3 * self.max_num_seqs_in_batch, self.max_decoding_seqs)
        if self.engine_prefill_chunk_size is None:
            self.engine_prefill_chunk_size = self.max_num_batched_tokens
        if self.engine_prefill_chunk_size <= 0:
            raise ValueError("engine_prefill_chunk_size must be positive")
        if self.mlp_chunk_size <= 0:
            raise ValueError("mlp_chunk_size must be positive")
        if self.state_slot_bytes < 0:
            raise ValueError("state_slot_bytes must not be negative")
        self.eos_token_ids = tuple(int(t) for t in self.eos_token_ids)
        if not isinstance(self.kernel_tuning, dict):
            raise ValueError("kernel_tuning must be a JSON object / dict")

    # Keys a tiny-random override file may shrink (src/sparseengine/debug/tiny_random.py:15-26).
    TINY_RANDOM_KEYS = ("head_dim", "hidden_size", "intermediate_size", "max_position_embeddings", "num_attention_heads",
                        "num_hidden_layers", "num_key_value_heads", "vocab_size")

    def apply_tiny_random_overrides(self, raw: dict) -> dict:
        """The model's config.json with the sizes of ``tiny_random_config`` put in, as the
        reference's tiny random mode does (src/sparseengine/debug/tiny_random.py:66-120): one
        JSON object of positive integers, only the keys above, present in the model's config,
        and the three main sizes never larger than the model's own."""
        if not self.tiny_random_config:
            return raw
        if not self.tiny_random:
            raise ValueError("tiny_random_config needs tiny_random=True")
        with open(self.tiny_random_config) as f:
            over = json.load(f)
        if not isinstance(over, dict):
            raise TypeError("the tiny random config must contain one JSON object")
        unknown = sorted(set(over) - set(self.TINY_RANDOM_KEYS))
        if unknown:
            raise ValueError(f"unsupported tiny random config keys: {unknown}; allowed: {sorted(self.TINY_RANDOM_KEYS)}")
        out = dict(raw)
        for k, v in over.items():
            if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
                raise ValueError(f"tiny random override {k} must be a positive integer, got {v!r}")
            if k not in raw:
                raise ValueError(f"tiny random override {k!r} is not a key of the model's config.json")
            if k in ("num_hidden_layers", "hidden_size", "intermediate_size") and v > int(raw[k]):
                raise ValueError(f"tiny random override {k} must not enlarge the model: {v} > {raw[k]}")
            out[k] = v
        return out

    @classmethod
    def field_names(cls) -> set:
        return {f.name for f in fields(cls)}

    @classmethod
    def from_kwargs(cls, model: str, **kwargs) -> "Config":
        unknown = sorted(set(kwargs) - cls.field_names())
        if unknown:
            raise ValueError(f"unknown engine option(s): {', '.join(unknown)}; known: {sorted(cls.field_names())}")
        return cls(model=model, **kwargs)

    @classmethod
    def from_json(cls, model: str, text_or_path: str) -> "Config":
        """``'{...}'`` or ``@file.json``, as the reference's ``--hyper_params``
        (benchmark/microbench.py:41-78)."""
        if text_or_path.startswith("@"):
            with open(text_or_path[1:]) as f:
                data = json.load(f)
        else:
            data = json.loads(text_or_path) if text_or_path else {}
        if not isinstance(data, dict):
            raise ValueError("hyper parameters must be a JSON object")
        return cls.from_kwargs(model, **data)
