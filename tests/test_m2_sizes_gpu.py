"""The engine at MiniMax M2's own layer sizes (two layers, random weights), around the sizes at
which one kernel hands over to another: the number of requests in a decode step and the
number of tokens in a prompt step.  The plain implementation would take minutes per case on a
CPU at these sizes, so the reference is the engine itself on another cut: a request's logits do
not depend on what else is in the step, and a prompt's logits at a position do not depend on how
many tokens follow it."""
import pytest
import torch

pytestmark = pytest.mark.gpu

M2_LAYER_SIZES = {
    "architectures": ["MiniMaxM2ForCausalLM"], "model_type": "minimax_m2", "num_hidden_layers": 2,
    "hidden_size": 3072, "num_attention_heads": 48, "num_key_value_heads": 8, "head_dim": 128,
    "rotary_dim": 64, "rope_theta": 5000000.0, "rms_norm_eps": 1e-6,
    "num_local_experts": 256, "num_experts_per_tok": 8, "intermediate_size": 1536,
    "vocab_size": 200064, "max_position_embeddings": 4096, "tie_word_embeddings": False,
    "hidden_act": "silu", "qk_norm_type": "per_layer", "use_qk_norm": True, "scoring_func": "sigmoid",
    "use_routing_bias": True, "use_mtp": True, "shared_intermediate_size": 0,
}
# bfloat16 logits here are below 8 in size, so one unit in the last place is 2^-5; up to 8 rows the
# dense projections take this library's kernel and beyond that the library product, whose sums differ
# in the last bit.  32-bit: only the order of sums differs.
TOL = {"bfloat16": 2 ** -5 + 1e-6, "float32": 3e-4}


@pytest.fixture(scope="module", params=["bfloat16", "float32"])
def engine(request):
    from sparseengine_b200 import LLM
    dtype = request.param
    llm = LLM(dict(M2_LAYER_SIZES, torch_dtype=dtype), tiny_random=True, tiny_random_seed=5, dtype=dtype,
              page_size=16, num_kvcache_slots=140 * 128, max_model_len=4096, max_num_seqs_in_gpu=140,
              max_num_seqs_in_batch=140, max_decoding_seqs=140, max_num_batched_tokens=8192)
    yield dtype, llm.runner
    del llm
    torch.cuda.empty_cache()


def test_a_request_decodes_the_same_beside_any_number_of_others(engine):
    from sparseengine_b200.csrc import ops
    from sparseengine_b200.engine.runner import StepEntry
    dtype, r = engine
    g = torch.Generator().manual_seed(1)
    n = 130
    prompts = [torch.randint(0, 200064, (int(torch.randint(3, 90, (1,), generator=g)),), generator=g).tolist()
               for _ in range(n)]
    nxt = [int(torch.randint(0, 200064, (1,), generator=g)) for _ in range(n)]
    alone = None
    for batch in (1, 2, 4, 5, 8, 9, 16, 17, 32, 33, 64, 65, 128, 129):
        ids = [(batch, i) for i in range(batch)]
        for sid in ids:
            r.admit(sid)
            r.step([StepEntry(sid, prompts[sid[1]], [])])
        logits = r.step([StepEntry(sid, [nxt[sid[1]]], [0]) for sid in ids]).float().cpu()
        ops.error_check("cuda:0")
        for sid in ids:
            r.release(sid)
        assert torch.isfinite(logits).all(), batch
        if alone is None:
            alone = logits[0]
        diff = (logits[0] - alone).abs().max().item()
        assert diff <= TOL[dtype], f"{dtype}: request 0 among {batch}: |diff| {diff:.3e}"
        if dtype == "bfloat16" and batch <= 8:
            assert diff == 0.0, f"request 0 among {batch}: the step's kernels are the same, the bits must be"


def test_a_prompt_gives_the_same_logits_whatever_its_length(engine):
    from sparseengine_b200.csrc import ops
    from sparseengine_b200.engine.runner import StepEntry
    dtype, r = engine
    g = torch.Generator().manual_seed(2)
    longest = 1100
    prompt = torch.randint(0, 200064, (longest,), generator=g).tolist()

    def run(sid, n):
        r.admit(sid)
        out = r.step([StepEntry(sid, prompt[:n], list(range(n)))]).float().cpu()
        r.release(sid)
        return out

    full = run("full", longest)
    for n in (1, 2, 4, 5, 8, 9, 16, 17, 32, 33, 64, 65, 127, 128, 129, 256, 257, 384, 385, 512, 513, 1024, 1025):
        got = run(f"n{n}", n)
        ops.error_check("cuda:0")
        assert torch.isfinite(got).all(), n
        diff = (got - full[:n]).abs().max().item()
        assert diff <= TOL[dtype], f"{dtype}: a prompt of {n} tokens against the first {n} of {longest}: |diff| {diff:.3e}"
