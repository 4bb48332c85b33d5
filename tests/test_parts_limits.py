"""Sizes a kernel cannot take are refused when the part is built, with the limit named, not at
the first step (no GPU needed: the parts only look at their spec)."""
import pytest
import torch

from sparseengine_b200.config.specs import AttentionSpec, MoESpec, RMSNormSpec, RotarySpec
from sparseengine_b200.csrc import ops
from sparseengine_b200.parts.base import make_feed_forward, make_mixer, make_norm


def test_norm_width():
    make_norm(RMSNormSpec(size=ops.LIMITS["rmsnorm_max_width"], eps=1e-6), torch.float32)
    with pytest.raises(ValueError, match="51200"):
        make_norm(RMSNormSpec(size=ops.LIMITS["rmsnorm_max_width"] + 1, eps=1e-6), torch.float32)
    with pytest.raises(ValueError, match="eps"):
        make_norm(RMSNormSpec(size=64, eps=0.0), torch.float32)


def test_attention_sizes():
    ok = dict(hidden_size=64, num_heads=4, num_kv_heads=2, head_dim=16, scale=0.25)
    make_mixer(AttentionSpec(**ok), torch.float32)
    for change, words in ((dict(head_dim=24), "head_dim"), (dict(head_dim=272), "head_dim"),
                          (dict(num_heads=5), "multiple"), (dict(num_heads=70000, num_kv_heads=1), "65535"),
                          (dict(window=0), "window"), (dict(qk_norm="per_head"), "qk_norm"),
                          (dict(position=RotarySpec(rotary_dim=32)), "rotates 32")):
        with pytest.raises(ValueError, match=words):
            make_mixer(AttentionSpec(**dict(ok, **change)), torch.float32)


def test_expert_counts_and_router_width():
    ok = dict(hidden_size=64, num_experts=8, top_k=2, intermediate_size=32)
    make_feed_forward(MoESpec(**ok), torch.float32)
    most = min(ops.LIMITS["router_max_experts"], ops.LIMITS["moe_max_experts"])
    make_feed_forward(MoESpec(**dict(ok, num_experts=most)), torch.float32)
    with pytest.raises(ValueError, match=str(most)):
        make_feed_forward(MoESpec(**dict(ok, num_experts=most + 1)), torch.float32)
    make_feed_forward(MoESpec(**dict(ok, hidden_size=7168)), torch.float32)          # a multiple of 4: any width
    with pytest.raises(ValueError, match="6400"):
        make_feed_forward(MoESpec(**dict(ok, hidden_size=6401)), torch.float32)
    with pytest.raises(ValueError, match="top_k"):
        make_feed_forward(MoESpec(**dict(ok, top_k=9)), torch.float32)


def test_a_step_cannot_have_more_entries_than_the_kernels_take():
    from sparseengine_b200.cache.manager import CacheManager
    from sparseengine_b200.config.registry import load_model_spec
    from sparseengine_b200.engine.model import Model
    from sparseengine_b200.engine.runner import ModelRunner
    import plain_m2
    from sparseengine_b200 import models  # noqa: F401
    _, spec = load_model_spec(plain_m2.TINY_A)
    m = Model(spec, torch.float32)
    cache = CacheManager(m.layout, page_size=4, num_pages=8, max_rows=70000, max_seq_len=64, allocate=False)
    with pytest.raises((ValueError, RuntimeError), match="65535|CUDA"):
        ModelRunner(m, cache, "cuda:0")
