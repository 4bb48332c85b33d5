"""Weights: load by tensor name, packed parameters, one error for everything wrong,
random-weights folders."""
import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

import plain_m2
import trace_util as tu
from sparseengine_b200 import models  # noqa: F401
from sparseengine_b200.config.registry import load_model_spec
from sparseengine_b200.engine.model import Model
from sparseengine_b200.weights.loader import WeightLoadError, load_weights
from sparseengine_b200.weights.random_init import write_random_model


def _model(cfg, dtype=torch.float32):
    _, spec = load_model_spec(cfg)
    return Model(spec, dtype)


@pytest.mark.parametrize("name", ["A", "B"])
def test_load_by_name_packs_qkv_and_experts(tmp_path, name):
    cfg = tu.TINY[name][0]
    tensors = tu.make_model_folder(str(tmp_path), name)
    m = _model(cfg)
    rep = load_weights(m, str(tmp_path), "cpu")
    assert rep.loaded == len(tensors) and not rep.skipped
    hq, hkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    inter = cfg["intermediate_size"]
    att = m.blocks[1].mixer
    p = "model.layers.1.self_attn."
    assert torch.equal(att.qkv[:hq * d], tensors[p + "q_proj.weight"])
    assert torch.equal(att.qkv[hq * d:(hq + hkv) * d], tensors[p + "k_proj.weight"])
    assert torch.equal(att.qkv[(hq + hkv) * d:], tensors[p + "v_proj.weight"])
    assert torch.equal(att.o, tensors[p + "o_proj.weight"])
    assert torch.equal(att.q_norm, tensors[p + "q_norm.weight"])
    ff = m.blocks[0].feed_forward
    q = "model.layers.0.block_sparse_moe."
    e = cfg["num_local_experts"] - 1
    assert torch.equal(ff.w13[e, :inter], tensors[f"{q}experts.{e}.w1.weight"])      # gate rows first
    assert torch.equal(ff.w13[e, inter:], tensors[f"{q}experts.{e}.w3.weight"])      # then up rows
    assert torch.equal(ff.w2[e], tensors[f"{q}experts.{e}.w2.weight"])
    assert torch.equal(ff.selection_bias, tensors[q + "e_score_correction_bias"])
    assert torch.equal(m.embed, tensors["model.embed_tokens.weight"])
    assert torch.equal(m.head, tensors["lm_head.weight"])


def test_bfloat16_engine_keeps_router_in_32_bit(tmp_path):
    tu.make_model_folder(str(tmp_path), "A", "bfloat16")
    m = _model(plain_m2.TINY_A, torch.bfloat16)
    load_weights(m, str(tmp_path), "cpu")
    assert m.blocks[0].mixer.qkv.dtype == torch.bfloat16
    assert m.blocks[0].feed_forward.gate.dtype == torch.float32
    assert m.blocks[0].feed_forward.selection_bias.dtype == torch.float32
    assert m.blocks[0].feed_forward.w13.dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    tensors = tu.make_model_folder(str(tmp_path), "A")
    path = os.path.join(str(tmp_path), "model.safetensors")
    t = dict(tensors)
    del t["model.layers.0.self_attn.k_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(4)
    t["lm_head.weight"] = torch.zeros(7, 3)
    t["model.layers.1.block_sparse_moe.experts.2.w2.weight"] = torch.zeros(5, 5)
    save_file(t, path)
    with pytest.raises(WeightLoadError) as e:
        load_weights(_model(plain_m2.TINY_A), str(tmp_path), "cpu")
    err = e.value
    assert set(err.missing) == {"model.layers.0.self_attn.k_proj.weight", "model.norm.weight"}
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert {n for n, _, _ in err.wrong_shape} == {"lm_head.weight",
                                                  "model.layers.1.block_sparse_moe.experts.2.w2.weight"}
    msg = str(err)
    for piece in ("k_proj", "model.norm.weight", "inv_freq", "lm_head.weight", "(7, 3)", "(256, 64)"):
        assert piece in msg


def test_mtp_tensors_are_skipped_and_counted(tmp_path):
    tensors = tu.make_model_folder(str(tmp_path), "A")
    t = dict(tensors)
    t["model.layers.2.self_attn.q_proj.weight"] = torch.zeros(3, 3)     # layer index == num_hidden_layers: MTP
    t["model.mtp_modules.0.norm.weight"] = torch.zeros(3)
    save_file(t, os.path.join(str(tmp_path), "model.safetensors"))
    rep = load_weights(_model(plain_m2.TINY_A), str(tmp_path), "cpu")
    assert sorted(rep.skipped) == ["model.layers.2.self_attn.q_proj.weight", "model.mtp_modules.0.norm.weight"]


def test_mtp_rule_follows_the_layer_index_and_the_stated_number_of_modules(tmp_path):
    """A tensor of ``model.layers.<i>.`` with i past the layers is a multi-token-prediction
    tensor whatever i is; when config.json states ``num_mtp_modules`` an index past those
    modules is not explained by the configuration and is reported as unexpected."""
    tensors = tu.make_model_folder(str(tmp_path), "A")
    t = dict(tensors)
    t["model.layers.40.mlp.w.weight"] = torch.zeros(2)
    save_file(t, os.path.join(str(tmp_path), "model.safetensors"))
    rep = load_weights(_model(plain_m2.TINY_A), str(tmp_path), "cpu")
    assert rep.skipped == ["model.layers.40.mlp.w.weight"]
    with pytest.raises(WeightLoadError) as e:
        load_weights(_model(dict(plain_m2.TINY_A, num_mtp_modules=3)), str(tmp_path), "cpu")
    assert e.value.unexpected == ["model.layers.40.mlp.w.weight"]
    t["model.layers.4.mlp.w.weight"] = t.pop("model.layers.40.mlp.w.weight")
    save_file(t, os.path.join(str(tmp_path), "model.safetensors"))
    rep = load_weights(_model(dict(plain_m2.TINY_A, num_mtp_modules=3)), str(tmp_path), "cpu")
    assert rep.skipped == ["model.layers.4.mlp.w.weight"]


def test_sharded_checkpoint_and_duplicates(tmp_path):
    tensors = tu.make_model_folder(str(tmp_path), "A")
    os.remove(os.path.join(str(tmp_path), "model.safetensors"))
    names = sorted(tensors)
    save_file({n: tensors[n] for n in names[:20]}, os.path.join(str(tmp_path), "model-00001-of-00002.safetensors"))
    save_file({n: tensors[n] for n in names[20:]}, os.path.join(str(tmp_path), "model-00002-of-00002.safetensors"))
    m = _model(plain_m2.TINY_A)
    assert load_weights(m, str(tmp_path), "cpu").loaded == len(tensors)
    save_file({names[0]: tensors[names[0]]}, os.path.join(str(tmp_path), "model-extra.safetensors"))
    with pytest.raises(WeightLoadError, match="more than one file"):
        load_weights(_model(plain_m2.TINY_A), str(tmp_path), "cpu")


def test_no_safetensors(tmp_path):
    with pytest.raises(FileNotFoundError):
        load_weights(_model(plain_m2.TINY_A), str(tmp_path), "cpu")


def test_random_weights_folder_is_seeded_and_loadable(tmp_path):
    a, b, c = (str(tmp_path / x) for x in "abc")
    write_random_model(a, plain_m2.TINY_B, seed=5, std=0.03, bias_std=0.1)
    write_random_model(b, plain_m2.TINY_B, seed=5, std=0.03, bias_std=0.1)
    write_random_model(c, plain_m2.TINY_B, seed=6, std=0.03, bias_std=0.1, dtype="bfloat16")
    ta, tb, tc = (load_file(os.path.join(x, "model.safetensors")) for x in (a, b, c))
    assert set(ta) == set(plain_m2.random_tensors(plain_m2.TINY_B, 0))
    assert all(torch.equal(ta[k], tb[k]) for k in ta)
    assert not torch.equal(ta["lm_head.weight"], tc["lm_head.weight"].float())
    assert tc["lm_head.weight"].dtype == torch.bfloat16
    assert tc["model.layers.0.block_sparse_moe.gate.weight"].dtype == torch.float32
    w = ta["model.embed_tokens.weight"]
    assert abs(float(w.std()) - 0.03) < 0.003
    assert abs(float(ta["model.layers.0.input_layernorm.weight"].mean()) - 1.0) < 1e-6
    cfg = json.load(open(os.path.join(a, "config.json")))
    assert cfg["architectures"] == ["MiniMaxM2ForCausalLM"]
    m = _model(cfg)
    assert load_weights(m, a, "cpu").loaded == len(ta)
    # the plain implementation runs on such a folder
    out = plain_m2.forward(cfg, ta, [1, 2, 3])
    assert out.shape == (3, cfg["vocab_size"]) and torch.isfinite(out).all()


def test_truncated_file_is_named(tmp_path):
    cfg = tu.TINY["A"][0]
    tu.make_model_folder(str(tmp_path), "A")
    path = os.path.join(str(tmp_path), "model.safetensors")
    size = os.path.getsize(path)
    with open(path, "r+b") as f:
        f.truncate(size // 2)
    with pytest.raises(WeightLoadError) as e:
        load_weights(_model(cfg), str(tmp_path), "cpu")
    assert "model.safetensors" in str(e.value) and "cannot be read" in str(e.value)
