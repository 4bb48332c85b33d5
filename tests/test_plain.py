"""The plain implementation itself: against SparseEngine's own CPU code where that can
run (tests/golden), and against properties the formulas imply."""
import os

import pytest
import torch
from safetensors.torch import load_file

import plain_m2

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "m2_front_end.safetensors")
ORACLES = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "m2_oracles.safetensors")


@pytest.mark.parametrize("name,cfg", [("A", plain_m2.TINY_A), ("B", plain_m2.TINY_B), ("C", plain_m2.TINY_C)])
def test_qk_norm_and_partial_rotary_match_the_reference_cpu_code(name, cfg):
    g = load_file(GOLDEN)
    hq, hkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps, rot, theta = cfg["rms_norm_eps"], cfg["rotary_dim"], cfg["rope_theta"]
    q, k, pos = g[f"{name}.q"], g[f"{name}.k"], g[f"{name}.positions"].long()
    qn = plain_m2.whole_projection_rms_norm(q, g[f"{name}.qw"], eps, torch.float32)
    kn = plain_m2.whole_projection_rms_norm(k, g[f"{name}.kw"], eps, torch.float32)
    assert torch.equal(qn, g[f"{name}.q_normed"]) and torch.equal(kn, g[f"{name}.k_normed"])
    t = q.shape[0]
    qo = plain_m2.partial_rotary(qn.view(t, hq, d), pos, rot, theta, torch.float32)
    ko = plain_m2.partial_rotary(kn.view(t, hkv, d), pos, rot, theta, torch.float32)
    assert torch.equal(qo, g[f"{name}.q_out"]) and torch.equal(ko, g[f"{name}.k_out"])
    if rot < d:     # pass-through dims are bit-equal to the normed values
        assert torch.equal(qo[..., rot:], qn.view(t, hq, d)[..., rot:])


def test_greedy_matches_the_reference_sampler():
    g = load_file(GOLDEN)
    assert torch.equal(g["sampler.logits"].argmax(-1).float(), g["sampler.greedy"])
    assert int(g["sampler.greedy"][2]) == 40


def test_router_order_and_weights():
    torch.manual_seed(0)
    x = torch.randn(5, 16)
    w = torch.randn(8, 16)
    bias = torch.randn(8) * 0.2
    ids, wt, logits = plain_m2.router(x, w, bias, 3)
    p = torch.sigmoid(logits)
    ref = torch.topk(p + bias, 3).indices
    for i in range(5):
        assert sorted(ids[i].tolist()) == sorted(ref[i].tolist())
        head = ids[i, :-1].tolist()                              # strictly above the k-th value: ascending index
        assert head == sorted(head)
        assert int(ids[i, -1]) == int(ref[i, -1])               # the k-th value itself comes last
        sel = p[i, ids[i]]
        assert torch.allclose(wt[i], sel / sel.sum())            # unbiased scores, renormalised
    # ties with the k-th value come after the strictly greater ones, by ascending index
    x1 = torch.zeros(1, 4)
    ids, wt, _ = plain_m2.router(x1, torch.zeros(6, 4), torch.tensor([0.0, 0.3, 0.0, 0.5, 0.0, 0.3]), 4)
    assert ids[0].tolist() == [1, 3, 5, 0]
    assert torch.allclose(wt[0], torch.full((4,), 0.25))


def test_experts_equal_a_dense_loop():
    torch.manual_seed(1)
    e, h, i, t, k = 5, 12, 7, 4, 2
    x = torch.randn(t, h)
    w1, w3, w2 = torch.randn(e, i, h) * 0.3, torch.randn(e, i, h) * 0.3, torch.randn(e, h, i) * 0.3
    ids = torch.tensor([[0, 1], [1, 4], [2, 3], [4, 0]])
    wt = torch.rand(t, k)
    out = plain_m2.experts(x, ids, wt, w1, w3, w2, torch.float32)
    ref = torch.zeros(t, h)
    for a in range(t):
        for s in range(k):
            ex = ids[a, s]
            ref[a] += wt[a, s] * (w2[ex] @ (torch.nn.functional.silu(w1[ex] @ x[a]) * (w3[ex] @ x[a])))
    assert torch.allclose(out, ref, atol=1e-5)


@pytest.mark.parametrize("cfg,seed", [(plain_m2.TINY_A, 0), (plain_m2.TINY_B, 1)])
def test_forward_is_causal_and_deterministic(cfg, seed):
    tensors = plain_m2.random_tensors(cfg, seed, 0.05, 0.05, 0.1)
    a = [3, 1, 4, 1, 5, 9, 2, 6]
    b = a[:5] + [7, 7, 7]
    la, lb = plain_m2.forward(cfg, tensors, a), plain_m2.forward(cfg, tensors, b)
    assert la.shape == (8, cfg["vocab_size"])
    # a position does not see later tokens (equal up to the order of sums: tokens that chose the
    # same expert go through one matrix product, whose blocking depends on how many they are)
    assert torch.allclose(la[:5], lb[:5], atol=1e-6, rtol=0)
    assert not torch.allclose(la[5:], lb[5:])
    assert torch.equal(la, plain_m2.forward(cfg, tensors, a))


def test_attention_window_and_groups():
    torch.manual_seed(2)
    t, hq, hkv, d = 9, 4, 2, 8
    q, k, v = torch.randn(t, hq, d), torch.randn(t, hkv, d), torch.randn(t, hkv, d)
    full = plain_m2.causal_attention(q, k, v, torch.float32)
    # first position attends to itself only
    assert torch.allclose(full[0, 0], v[0, 0]) and torch.allclose(full[0, 3], v[0, 1])
    w = plain_m2.causal_attention(q, k, v, torch.float32, window=3)
    assert torch.allclose(w[:3], full[:3]) and not torch.allclose(w[5], full[5])
    s = (q[6, 1] @ k[4:7, 0].t()) * d ** -0.5
    assert torch.allclose(w[6, 1], torch.softmax(s, -1) @ v[4:7, 0], atol=1e-6)


def test_bfloat16_rounding_points_are_bfloat16_values():
    cfg = plain_m2.TINY_A
    tensors = plain_m2.random_tensors(cfg, 0, 0.05, 0.05)
    out = plain_m2.forward(cfg, tensors, [1, 2, 3, 4], torch.bfloat16)
    assert torch.equal(out, out.to(torch.bfloat16).float())
    ref = plain_m2.forward(cfg, tensors, [1, 2, 3, 4])
    assert (out - ref).abs().max() < 0.05


# ---- the reference's own pure-torch oracles (tests/golden/make_golden.py wrote their outputs) ----

def test_rms_norm_matches_the_reference_oracle():
    g = load_file(ORACLES)
    x, w = g["rmsnorm.x"], g["rmsnorm.w"]
    assert torch.allclose(plain_m2.rms_norm(x, w, 1e-5, torch.float32), g["rmsnorm.f32"], atol=0, rtol=2e-7)
    got = plain_m2.rms_norm(x.bfloat16().float(), w.bfloat16().float(), 1e-5, torch.bfloat16)
    assert torch.equal(got, g["rmsnorm.bf16"])


def test_router_matches_the_reference_oracle_at_m2_size():
    """256 experts, top-8: the same experts and, expert by expert, the same weights (the oracle
    returns them in the order of an unsorted top-k; the order rule of the kernels, strictly
    greater first and ties by ascending index, is checked in test_router_order_and_weights)."""
    g = load_file(ORACLES)
    logits, bias = g["router.logits"], g["router.bias"]
    want_ids, want_w = g["router.ids"].long(), g["router.weights"]
    # the plain router takes activations and a gate: feed the logits through an identity gate
    ids, w, got_logits = plain_m2.router(logits, torch.eye(256), bias, 8)
    assert torch.equal(got_logits, logits)
    for t in range(logits.shape[0]):
        assert sorted(ids[t].tolist()) == sorted(want_ids[t].tolist()), t
        mine = dict(zip(ids[t].tolist(), w[t].tolist()))
        for e, x in zip(want_ids[t].tolist(), want_w[t].tolist()):
            assert abs(mine[e] - x) <= 2e-7, (t, e)


def test_experts_match_the_reference_oracle():
    g = load_file(ORACLES)
    inter = g["moe.w2"].shape[2]
    out = plain_m2.experts(g["moe.x"], g["moe.ids"].long(), g["moe.weights"], g["moe.w13"][:, :inter],
                           g["moe.w13"][:, inter:], g["moe.w2"], torch.float32)
    assert torch.allclose(out, g["moe.out"], atol=2e-6, rtol=1e-5)


def test_sampling_cuts_keep_what_the_reference_sampler_can_draw():
    from golden.golden_cases import SAMPLER_CASES
    g = load_file(ORACLES)
    row = g["sampler.row"]
    sizes = []
    for i, (top_k, top_p, temp) in enumerate(SAMPLER_CASES):
        kept = plain_m2.sampling_kept(row, top_k, top_p, temp)
        support = g[f"sampler.support.{i}"].bool()
        assert not (support & ~kept).any(), (i, "the reference drew a token the plain cuts remove")
        # every kept token with a chance of at least one in a thousand shows up in 6,000 draws
        p = torch.softmax(torch.where(kept, row / temp, torch.tensor(float("-inf"))), -1)
        assert not (kept & ~support & (p > 1e-3)).any(), (i, "the plain cuts keep a token the reference never draws")
        sizes.append(int(kept.sum()))
    assert sizes[0] == 40 and sizes[1] == 5 and sizes[-1] == 1 and 1 < sizes[3] <= 8


def test_scaled_rotary_frequencies_match_the_reference():
    from golden.golden_cases import ROPE_SCALINGS
    g = load_file(ORACLES)
    for name, scaling in ROPE_SCALINGS.items():
        inv, factor = plain_m2.rope_frequencies(64, 5e6, scaling)
        assert torch.allclose(inv, g[f"rope.{name}.inv_freq"], atol=0, rtol=2e-6), name
        assert abs(factor - float(g[f"rope.{name}.factor"])) < 1e-6, name
    assert float(g["rope.yarn_factor.factor"]) == 1.25 and float(g["rope.linear.factor"]) == 1.0


def test_rotation_of_adjacent_pairs_matches_the_reference():
    g = load_file(ORACLES)
    x, ang = g["interleaved.x"], g["interleaved.angle"]
    # positions and frequencies whose products are the stored angles: position p, frequency angle/p
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., 0::2], x[..., 1::2]
    want = torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), -1)
    assert torch.equal(want, g["interleaved.out"])
    pos = torch.tensor([0, 1, 2, 7, 300])
    got = plain_m2.partial_rotary(x, pos, 16, 10000.0, torch.float32, interleaved=True)
    assert torch.allclose(got, g["interleaved.out"], atol=2e-6)
