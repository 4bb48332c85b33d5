"""MiniMax M2 (``MiniMaxM2ForCausalLM``): typed configuration and model description.

Every layer: RMSNorm → grouped-query attention with a whole-projection QK RMSNorm and a
partial rotary encoding → RMSNorm → routed SwiGLU experts (sigmoid scores, selection
bias, renormalised top-k).  No shared expert, no window; multi-token-prediction tensors
in a checkpoint are skipped.

Reference: src/sparseengine/models/minimax_m2.py:140-172 (router), :175-209 (experts),
:272-359 (attention), :362-397 (layer), :417-423,513-530 (tensor names);
src/sparseengine/models/checkpoint.py:222-244 (accepted option values);
src/sparseengine/models/rope.py:37-43 (rope_theta), src/sparseengine/configs/model.py:29-35
(context-length keys).
"""
from __future__ import annotations

import re
from dataclasses import dataclass, fields
from typing import Optional

from ..config.registry import register_architecture
from ..config.specs import (AttentionSpec, LayerSpec, ModelSpec, MoESpec, RMSNormSpec,
                            RotarySpec, ScheduleEntry, Source)

ARCHITECTURE = "MiniMaxM2ForCausalLM"

_CONTEXT_LENGTH_KEYS = ("max_sequence_length", "seq_length", "max_seq_len",
                        "model_max_length", "max_position_embeddings")

# Option values the architecture is defined for; another value is refused, an absent
# key takes the value shown.
_REQUIRED_OPTIONS = {
    "hidden_act": "silu",
    "qk_norm_type": "per_layer",
    "scoring_func": "sigmoid",
    "use_qk_norm": True,
    "use_routing_bias": True,
    "tie_word_embeddings": False,
}


@dataclass(frozen=True)
class MiniMaxM2Config:
    """The ``config.json`` keys MiniMax M2 is built from.  No size has a default."""
    vocab_size: int
    hidden_size: int
    intermediate_size: int            # per-expert SwiGLU width
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rotary_dim: int
    num_local_experts: int
    num_experts_per_tok: int
    max_position_embeddings: int
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    shared_intermediate_size: int = 0
    rope_scaling: Optional[tuple] = None     # sorted (key, value) pairs of a linear / llama3 / yarn frequency scaling
    num_mtp_modules: Optional[int] = None    # multi-token-prediction modules stored after the layers (None: not stated)
    stored_dtype: str = "bfloat16"
    model_type: str = "minimax_m2"

    @classmethod
    def from_dict(cls, raw: dict) -> "MiniMaxM2Config":
        problems = []
        for key, want in _REQUIRED_OPTIONS.items():
            if key in raw and raw[key] != want:
                problems.append(f"{key}={raw[key]!r} (only {want!r} is supported)")
        if raw.get("quantization_config"):
            problems.append("quantization_config is set (quantized weights are not supported)")
        if int(raw.get("shared_intermediate_size", 0) or 0) != 0:
            problems.append("shared_intermediate_size != 0 (M2 has no shared expert)")
        # frequency scaling: ``rope_parameters`` if it is there, else ``rope_scaling``
        # (src/sparseengine/models/rope.py:14-35); linear, llama3 and yarn become a frequency table
        # built on the host, the types that depend on the sequence length are refused (:77-88)
        params = dict(raw.get("rope_parameters") or raw.get("rope_scaling") or {})
        rope_type = str(params.get("rope_type", params.get("type", "default")) or "default").lower()
        params.pop("type", None)
        rope_scaling = None
        if rope_type in ("linear", "llama3", "yarn"):
            params["rope_type"] = rope_type
            rope_scaling = tuple(sorted((k, tuple(v) if isinstance(v, list) else v) for k, v in params.items()
                                        if k != "rope_theta"))
        elif rope_type != "default":
            problems.append(f"rope scaling type {rope_type!r} (default, linear, llama3 and yarn are supported)")

        required = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim", "rotary_dim",
                    "num_local_experts", "num_experts_per_tok")
        missing = [k for k in required if raw.get(k) is None]
        if missing:
            problems.append("missing keys: " + ", ".join(missing))
        max_pos = None
        for key in _CONTEXT_LENGTH_KEYS:
            if raw.get(key) is not None:
                max_pos = int(raw[key])
                break
        if max_pos is None:
            problems.append("no context length key (" + ", ".join(_CONTEXT_LENGTH_KEYS) + ")")
        if problems:
            raise ValueError("MiniMax M2 config.json cannot be used: " + "; ".join(problems))

        theta = params.get("rope_theta", raw.get("rope_theta", 10000.0))
        dtype = raw.get("dtype", raw.get("torch_dtype", "bfloat16"))
        cfg = cls(
            vocab_size=int(raw["vocab_size"]), hidden_size=int(raw["hidden_size"]),
            intermediate_size=int(raw["intermediate_size"]),
            num_hidden_layers=int(raw["num_hidden_layers"]),
            num_attention_heads=int(raw["num_attention_heads"]),
            num_key_value_heads=int(raw["num_key_value_heads"]),
            head_dim=int(raw["head_dim"]), rotary_dim=int(raw["rotary_dim"]),
            num_local_experts=int(raw["num_local_experts"]),
            num_experts_per_tok=int(raw["num_experts_per_tok"]),
            max_position_embeddings=max_pos, rope_theta=float(theta),
            rms_norm_eps=float(raw.get("rms_norm_eps", 1e-6)), rope_scaling=rope_scaling,
            num_mtp_modules=None if raw.get("num_mtp_modules") is None else int(raw["num_mtp_modules"]),
            stored_dtype=str(dtype).replace("torch.", ""),
            model_type=str(raw.get("model_type", "minimax_m2")),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        bad = []
        for f in fields(self):
            v = getattr(self, f.name)
            if f.type in (int, "int") and f.name != "shared_intermediate_size" and v <= 0:
                bad.append(f"{f.name}={v} must be positive")
        if self.num_attention_heads % max(self.num_key_value_heads, 1):
            bad.append("num_attention_heads must be a multiple of num_key_value_heads")
        if self.rotary_dim > self.head_dim or self.rotary_dim % 2:
            bad.append("rotary_dim must be even and at most head_dim")
        if self.num_experts_per_tok > self.num_local_experts:
            bad.append("num_experts_per_tok exceeds num_local_experts")
        if not (self.rope_theta > 0) or not (self.rms_norm_eps > 0):
            bad.append("rope_theta and rms_norm_eps must be positive")
        if self.rope_scaling is not None:
            from ..parts.position import scaled_frequencies
            try:
                scaled_frequencies(self.rotary_dim, self.rope_theta, dict(self.rope_scaling))
            except ValueError as e:
                bad.append(str(e))
        if bad:
            raise ValueError("MiniMax M2 config.json cannot be used: " + "; ".join(bad))

    def to_dict(self) -> dict:
        """A ``config.json`` dictionary that reads back to this configuration."""
        out = {
            "architectures": [ARCHITECTURE], "model_type": self.model_type,
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim, "rotary_dim": self.rotary_dim,
            "rope_theta": self.rope_theta, "rms_norm_eps": self.rms_norm_eps,
            "num_local_experts": self.num_local_experts,
            "num_experts_per_tok": self.num_experts_per_tok,
            "max_position_embeddings": self.max_position_embeddings,
            "shared_intermediate_size": 0, "torch_dtype": self.stored_dtype,
        }
        out.update(_REQUIRED_OPTIONS)
        out["use_mtp"] = True
        if self.num_mtp_modules is not None:
            out["num_mtp_modules"] = self.num_mtp_modules
        if self.rope_scaling is not None:
            out["rope_scaling"] = {k: list(v) if isinstance(v, tuple) else v for k, v in self.rope_scaling}
        return out


_LAYER_INDEX = re.compile(r"^model\.layers\.(\d+)\.")


def mtp_tensor_rule(num_layers: int, num_mtp_modules: Optional[int]):
    """Which checkpoint tensors belong to multi-token-prediction modules: those stored as
    further decoder layers, ``model.layers.<i>.`` with ``num_layers <= i`` (and, when the
    configuration states how many modules there are, ``i < num_layers + num_mtp_modules``:
    an index beyond that is not explained by the configuration and stays an error)."""
    def rule(name: str) -> bool:
        m = _LAYER_INDEX.match(name)
        if m is None:
            return False
        i = int(m.group(1))
        if i < num_layers:
            return False
        return num_mtp_modules is None or i < num_layers + num_mtp_modules
    return rule


def build_minimax_m2(cfg: MiniMaxM2Config) -> ModelSpec:
    h, d = cfg.hidden_size, cfg.head_dim
    hq, hkv = cfg.num_attention_heads, cfg.num_key_value_heads
    e, inter = cfg.num_local_experts, cfg.intermediate_size
    rotary = RotarySpec(rotary_dim=cfg.rotary_dim, theta=cfg.rope_theta, frequency_scaling=cfg.rope_scaling)
    attention = AttentionSpec(
        hidden_size=h, num_heads=hq, num_kv_heads=hkv, head_dim=d, scale=d ** -0.5,
        qk_norm="whole_projection", qk_norm_eps=cfg.rms_norm_eps, window=None, position=rotary)
    moe = MoESpec(hidden_size=h, num_experts=e, top_k=cfg.num_experts_per_tok,
                  intermediate_size=inter, score_fn="sigmoid", selection_bias=True,
                  renormalize=True, routed_scale=1.0, activation="silu")
    norm = RMSNormSpec(size=h, eps=cfg.rms_norm_eps)

    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        a = p + "self_attn."
        m = p + "block_sparse_moe."
        w13, w2 = [], []
        for j in range(e):
            x = f"{m}experts.{j}."
            # w1 = gate rows first, then w3 = up rows; w2 = down.
            w13.append(Source(x + "w1.weight", (j, (0, inter))))
            w13.append(Source(x + "w3.weight", (j, (inter, inter))))
            w2.append(Source(x + "w2.weight", (j,)))
        sources = {
            "mixer_norm.weight": (Source(p + "input_layernorm.weight"),),
            "feed_forward_norm.weight": (Source(p + "post_attention_layernorm.weight"),),
            "mixer.qkv": (Source(a + "q_proj.weight", ((0, hq * d),)),
                          Source(a + "k_proj.weight", ((hq * d, hkv * d),)),
                          Source(a + "v_proj.weight", ((hq * d + hkv * d, hkv * d),))),
            "mixer.o": (Source(a + "o_proj.weight"),),
            "mixer.q_norm": (Source(a + "q_norm.weight"),),
            "mixer.k_norm": (Source(a + "k_norm.weight"),),
            "feed_forward.gate": (Source(m + "gate.weight"),),
            "feed_forward.selection_bias": (Source(m + "e_score_correction_bias"),),
            "feed_forward.w13": tuple(w13),
            "feed_forward.w2": tuple(w2),
        }
        layers.append(LayerSpec(mixer=attention, feed_forward=moe, mixer_norm=norm,
                                feed_forward_norm=norm, sources=sources))
    order = [ScheduleEntry(layer=i) for i in range(cfg.num_hidden_layers)]
    # Multi-token-prediction modules live outside model.layers.[0, L); the model has no
    # use for them, so their tensors are skipped and counted at load.
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=h, vocab_size=cfg.vocab_size,
        max_position=cfg.max_position_embeddings, layers=layers, order=order,
        final_norm=norm, embed_source="model.embed_tokens.weight", head_source="lm_head.weight",
        ignored_prefixes=("model.mtp", "mtp.", "model.mtp_modules"),
        ignored_rule=mtp_tensor_rule(cfg.num_hidden_layers, cfg.num_mtp_modules),
        stored_dtype=cfg.stored_dtype)


register_architecture(ARCHITECTURE, MiniMaxM2Config, build_minimax_m2)
