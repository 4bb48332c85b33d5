"""Configuration: the architecture's typed config, the registry, engine options."""
import json

import pytest

import plain_m2
from sparseengine_b200 import models  # noqa: F401
from sparseengine_b200.config.engine_config import Config
from sparseengine_b200.config.registry import architectures, load_model_spec
from sparseengine_b200.models.minimax_m2 import MiniMaxM2Config


@pytest.mark.parametrize("cfg", [plain_m2.TINY_A, plain_m2.TINY_B, plain_m2.TINY_C])
def test_m2_config_reads_every_size(cfg):
    typed, spec = load_model_spec(cfg)
    assert isinstance(typed, MiniMaxM2Config)
    assert spec.vocab_size == cfg["vocab_size"] and spec.hidden_size == cfg["hidden_size"]
    assert len(spec.layers) == cfg["num_hidden_layers"] == len(spec.order)
    a = spec.layers[0].mixer
    assert (a.num_heads, a.num_kv_heads, a.head_dim) == (cfg["num_attention_heads"], cfg["num_key_value_heads"],
                                                          cfg["head_dim"])
    assert a.position.rotary_dim == cfg["rotary_dim"] and a.position.theta == cfg["rope_theta"]
    assert a.qk_norm == "whole_projection" and a.qk_norm_eps == cfg["rms_norm_eps"]
    assert a.scale == cfg["head_dim"] ** -0.5 and a.window is None
    f = spec.layers[-1].feed_forward
    assert (f.num_experts, f.top_k, f.intermediate_size) == (cfg["num_local_experts"], cfg["num_experts_per_tok"],
                                                             cfg["intermediate_size"])
    assert f.score_fn == "sigmoid" and f.selection_bias and f.renormalize
    assert spec.layers[0].mixer_norm.eps == cfg["rms_norm_eps"]
    assert typed.to_dict()["num_local_experts"] == cfg["num_local_experts"]
    assert MiniMaxM2Config.from_dict(typed.to_dict()) == typed


def test_m2_config_refuses_what_it_cannot_run():
    bad = dict(plain_m2.TINY_A, scoring_func="softmax", qk_norm_type="per_head")
    with pytest.raises(ValueError) as e:
        load_model_spec(bad)
    assert "scoring_func" in str(e.value) and "qk_norm_type" in str(e.value)
    missing = {k: v for k, v in plain_m2.TINY_A.items() if k not in ("rotary_dim", "head_dim")}
    with pytest.raises(ValueError) as e:
        load_model_spec(missing)
    assert "rotary_dim" in str(e.value) and "head_dim" in str(e.value)
    with pytest.raises(ValueError):
        load_model_spec(dict(plain_m2.TINY_A, num_attention_heads=5))
    with pytest.raises(ValueError):
        load_model_spec(dict(plain_m2.TINY_A, quantization_config={"quant_method": "fp8"}))
    with pytest.raises(ValueError):
        load_model_spec(dict(plain_m2.TINY_A, rope_scaling={"rope_type": "yarn", "factor": 2.0}))


def test_rope_theta_from_rope_parameters_and_context_keys():
    cfg = {k: v for k, v in plain_m2.TINY_A.items() if k not in ("rope_theta", "max_position_embeddings")}
    cfg["rope_parameters"] = {"rope_theta": 12345.0, "rope_type": "default"}
    cfg["max_seq_len"] = 77
    typed, spec = load_model_spec(cfg)
    assert typed.rope_theta == 12345.0 and spec.max_position == 77


def test_registry():
    assert "MiniMaxM2ForCausalLM" in architectures()
    with pytest.raises(ValueError, match="unknown architecture"):
        load_model_spec({"architectures": ["NoSuchModel"]})
    with pytest.raises(ValueError):
        load_model_spec({"architectures": []})


def test_engine_options(tmp_path):
    c = Config.from_kwargs("m", max_num_batched_tokens=128, max_num_seqs_in_batch=4)
    assert c.max_decoding_seqs == 4 and c.max_num_seqs_in_gpu == 12 and c.engine_prefill_chunk_size == 128
    with pytest.raises(ValueError, match="unknown engine option"):
        Config.from_kwargs("m", no_such_option=1)
    with pytest.raises(ValueError):
        Config.from_kwargs("m", sparse_method="snapkv")
    with pytest.raises(ValueError):
        Config.from_kwargs("m", tensor_parallel_size=2)
    assert Config.from_kwargs("m", sparse_method="vanilla").sparse_method == "vanilla"
    p = tmp_path / "hp.json"
    p.write_text(json.dumps({"page_size": 8, "dtype": "float32"}))
    c = Config.from_json("m", "@" + str(p))
    assert c.page_size == 8 and c.dtype == "float32"
    assert Config.from_json("m", '{"seed": 3}').seed == 3


def test_tiny_random_override_file(tmp_path):
    """The reference's tiny random mode: a JSON file that shrinks sizes of the model's config."""
    import json
    from sparseengine_b200.config.engine_config import Config
    raw = dict(plain_m2.TINY_A)
    path = tmp_path / "tiny.json"
    path.write_text(json.dumps({"num_hidden_layers": 1, "vocab_size": 99}))
    cfg = Config.from_kwargs("m", tiny_random=True, tiny_random_config=str(path))
    out = cfg.apply_tiny_random_overrides(raw)
    assert out["num_hidden_layers"] == 1 and out["vocab_size"] == 99 and raw["num_hidden_layers"] != 1
    assert Config.from_kwargs("m").apply_tiny_random_overrides(raw) is raw
    with pytest.raises(ValueError, match="tiny_random=True"):
        Config.from_kwargs("m", tiny_random_config=str(path)).apply_tiny_random_overrides(raw)
    for bad, msg in (({"num_experts_per_tok": 1}, "unsupported"), ({"hidden_size": 0}, "positive"),
                     ({"hidden_size": 10 ** 6}, "enlarge"), ({"num_hidden_layers": True}, "positive")):
        path.write_text(json.dumps(bad))
        with pytest.raises(ValueError, match=msg):
            cfg.apply_tiny_random_overrides(raw)


def test_scaled_rotary_tables_are_built_on_the_host_and_match_the_reference():
    """linear / llama3 / yarn frequency scaling becomes a table of frequencies and a factor on
    cos and sin: compared with the tables the reference's own code gave (tests/golden)."""
    import os

    import torch
    from safetensors.torch import load_file

    from golden.golden_cases import ROPE_SCALINGS
    from sparseengine_b200.config.specs import RotarySpec
    from sparseengine_b200.parts.base import make_position
    from sparseengine_b200.parts.position import scaled_frequencies
    g = load_file(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "m2_oracles.safetensors"))
    for name, scaling in ROPE_SCALINGS.items():
        inv, factor = scaled_frequencies(64, 5e6, scaling)
        assert torch.allclose(inv, g[f"rope.{name}.inv_freq"], atol=0, rtol=2e-6), name
        assert abs(factor - float(g[f"rope.{name}.factor"])) < 1e-6, name
    # through the configuration: a yarn entry in config.json reaches the attention part's position encoding
    cfg = dict(plain_m2.TINY_A, head_dim=64, rotary_dim=64, rope_theta=5e6, rope_scaling=ROPE_SCALINGS["yarn"])
    typed, spec = load_model_spec(cfg)
    pos = make_position(spec.layers[0].mixer.position, torch.float32)
    args = pos.kernel_args("cpu")
    assert torch.allclose(args.inv_freq, g["rope.yarn.inv_freq"], rtol=2e-6, atol=0)
    assert abs(args.scale - float(g["rope.yarn.factor"])) < 1e-6 and args.pairing == "split_half"
    assert load_model_spec(typed.to_dict())[0] == typed                 # and reads back from its own config.json
    for bad in ({"rope_type": "dynamic", "factor": 2.0}, {"rope_type": "yarn", "factor": 2.0},
                {"rope_type": "llama3", "factor": 2.0, "original_max_position_embeddings": 64, "low_freq_factor": 4.0,
                 "high_freq_factor": 1.0}, {"rope_type": "linear", "factor": 0.5}):
        with pytest.raises(ValueError):
            load_model_spec(dict(plain_m2.TINY_A, rope_scaling=bad))
    with pytest.raises(ValueError):
        make_position(RotarySpec(rotary_dim=24, pairing="pairs_of_three"), torch.float32)


def test_kernel_tuning_options_are_checked_and_reach_the_parts():
    import torch

    from sparseengine_b200.config.engine_config import Config
    from sparseengine_b200.engine.factory import KERNEL_TUNING_KEYS, apply_kernel_tuning, check_kernel_tuning
    from sparseengine_b200.engine.model import Model
    cfg = Config.from_kwargs("m", kernel_tuning={"attention_decode_kernel_max_tokens": 64, "moe_pair_min_rows": 4096})
    check_kernel_tuning(cfg.kernel_tuning)
    for bad in ({"no_such_threshold": 1}, {"attention_portion_min_tokens": -1}, {"gemv_max_out_features": 1.5}):
        with pytest.raises(ValueError):
            check_kernel_tuning(bad)
    with pytest.raises(ValueError):
        Config.from_kwargs("m", kernel_tuning=[1, 2])
    _, spec = load_model_spec(plain_m2.TINY_A)
    m = Model(spec, torch.float32)
    apply_kernel_tuning(m, cfg.kernel_tuning)
    assert all(b.mixer.decode_kernel_max_tokens == 64 and b.feed_forward.pair_min_rows == 4096 for b in m.blocks)
    from sparseengine_b200.parts import linear
    before = linear.GEMV_MAX_ROWS, linear.GEMV_MAX_OUT
    try:
        apply_kernel_tuning(m, {"gemv_max_rows": 3, "gemv_max_out_features": 100})
        assert (linear.GEMV_MAX_ROWS, linear.GEMV_MAX_OUT) == (3, 100)
    finally:
        linear.GEMV_MAX_ROWS, linear.GEMV_MAX_OUT = before
    assert set(KERNEL_TUNING_KEYS) >= {"router_tensor_core_min_tokens", "moe_pair_min_rows_per_expert"}
