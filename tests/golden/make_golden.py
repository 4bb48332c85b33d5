"""Golden outputs from CURRENTF/SparseEngine's own CPU code for the parts of MiniMax M2
that can run without CUDA: the whole-projection QK RMSNorm pair
(src/sparseengine/layers/layernorm.py:217-255), the partial rotary encoding
(src/sparseengine/layers/rotary_embedding.py:129-167 with the torch backend) and the
greedy branch of the sampler (src/sparseengine/layers/sampler.py:123-135).

The reference's RMSNorm, router and experts need CUDA + Triton and its whole model
cannot be built on a CPU, so those parts of tests/plain_m2.py rest on the formulas.

Run once, with the reference checkout importable:

    PYTHONPATH=<reference>/src SPARSEENGINE_PLATFORM=cpu CUDA_VISIBLE_DEVICES="" \
        python tests/golden/make_golden.py

It writes tests/golden/m2_front_end.safetensors (inputs and outputs, float32, a few KB),
which tests/test_plain.py compares with the plain implementation.
"""
import os
import sys

import torch
from safetensors.torch import save_file

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import plain_m2  # noqa: E402

from sparseengine.distributed import ParallelContext, ParallelGroup  # noqa: E402
from sparseengine.layers.layernorm import ColumnParallelRMSNorm  # noqa: E402
from sparseengine.layers.rotary_embedding import apply_partial_rotary_emb, apply_rotary_emb, get_rope  # noqa: E402
from sparseengine.layers.sampler import Sampler  # noqa: E402


def context():
    g = ParallelGroup(None, (0,), 0, 1)
    return ParallelContext(world=g, moe_tp=g, attn_tp=g, moe_ep=g, attn_dp=g)


def main():
    out = {}
    ctx = context()
    for name, cfg in (("A", plain_m2.TINY_A), ("B", plain_m2.TINY_B), ("C", plain_m2.TINY_C)):
        torch.manual_seed(11)
        hq, hkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        rot, theta, eps = cfg["rotary_dim"], cfg["rope_theta"], cfg["rms_norm_eps"]
        t = 7
        q = torch.randn(t, hq * d) * 3.0
        k = torch.randn(t, hkv * d) * 0.3
        qw = 1.0 + 0.1 * torch.randn(hq * d)
        kw = 1.0 + 0.1 * torch.randn(hkv * d)
        positions = torch.tensor([0, 1, 2, 5, 17, 100, 411])
        qn = ColumnParallelRMSNorm(hq * d, eps=eps, parallel_context=ctx)
        kn = ColumnParallelRMSNorm(hkv * d, eps=eps, parallel_context=ctx)
        with torch.no_grad():
            qn.weight.copy_(qw)
            kn.weight.copy_(kw)
            q1, k1 = qn.forward_pair(q, k, kn)
            rope = get_rope(rot, rotary_dim=rot, max_position=cfg["max_position_embeddings"], base=theta,
                            rope_scaling=None)
            rope.backend = "torch"
            q3, k3 = q1.view(t, hq, d), k1.view(t, hkv, d)
            if rot == d:
                cos, sin = rope.cos_sin_cache[positions].chunk(2, dim=-1)
                q2 = apply_rotary_emb(q3, cos, sin)      # the cache is [positions, 1, R]
                k2 = apply_rotary_emb(k3, cos, sin)
            else:
                q2, k2 = apply_partial_rotary_emb(rope, positions, q3, k3, rot)
        for key, val in (("q", q), ("k", k), ("qw", qw), ("kw", kw), ("positions", positions.float()),
                         ("q_normed", q1), ("k_normed", k1), ("q_out", q2), ("k_out", k2)):
            out[f"{name}.{key}"] = val.contiguous().float()
    torch.manual_seed(5)
    logits = torch.randn(6, 97)
    logits[2, 40] = logits[2, 41] = 9.0          # a tie: argmax takes the first
    out["sampler.logits"] = logits
    out["sampler.greedy"] = Sampler()(logits, None, all_greedy=True).float()
    save_file(out, os.path.join(HERE, "m2_front_end.safetensors"))
    print("wrote", len(out), "tensors")


if __name__ == "__main__":
    main()
