"""Scheduler decisions on the CPU, with the real cache manager (no storage) and a fake
step that "samples" token 7."""
import pytest

from sparseengine_b200.cache.manager import CacheManager
from sparseengine_b200.config.engine_config import Config
from sparseengine_b200.engine.model import CacheLayout, EntryCache
from sparseengine_b200.engine.scheduler import Scheduler
from sparseengine_b200.engine.sequence import Sequence
from sparseengine_b200.parts.base import KVRequest
from sparseengine_b200.sampling.params import SamplingParams


def make(num_pages=64, page_size=4, max_model_len=256, **opts):
    lay = CacheLayout(((KVRequest(2, 16, None), 1),), (), (EntryCache(0, 0, True, None),))
    cfg = Config.from_kwargs("m", page_size=page_size, **opts)
    cm = CacheManager(lay, page_size=page_size, num_pages=num_pages, max_rows=cfg.max_num_seqs_in_gpu,
                      max_seq_len=max_model_len, allocate=False)
    return Scheduler(cfg, cm, eos_token_ids=(99,), max_model_len=max_model_len), cm


def run_step(sched, cm, token=7, tokens=None):
    plan = sched.schedule()
    for it in plan.items:                       # what the step function does with the cache
        cm.reserve(it.seq.seq_id, it.n_tokens)
    for it in plan.items:
        cm.commit(it.seq.seq_id, it.n_tokens)
    n = sum(1 for it in plan.items if it.samples)
    out = tokens if tokens is not None else [token] * n
    return plan, sched.postprocess(plan, out[:n])


def seq(i, n, **sp):
    sp.setdefault("max_tokens", 4)
    return Sequence(i, list(range(1, n + 1)), SamplingParams(**sp))


def test_prompt_is_cut_under_the_token_budget_then_decodes():
    sched, cm = make(max_num_batched_tokens=8, max_num_seqs_in_batch=4)
    sched.add(seq(0, 19))
    sizes = []
    for _ in range(3):
        plan, fin = run_step(sched, cm)
        sizes.append([(it.start, it.n_tokens, it.samples) for it in plan.items])
    assert sizes == [[(0, 8, False)], [(8, 8, False)], [(16, 3, True)]]
    s = sched.running[0]
    assert s.output_ids == [7] and s.in_decode
    plan, _ = run_step(sched, cm)
    assert [(it.start, it.n_tokens) for it in plan.items] == [(19, 1)] and plan.num_decodes == 0 or True


def test_decodes_and_prompt_portions_share_a_step():
    sched, cm = make(max_num_batched_tokens=10, max_num_seqs_in_batch=4)
    sched.add(seq(0, 3, max_tokens=8))
    run_step(sched, cm)                          # request 0 prefills whole, now decodes
    sched.add(seq(1, 20, max_tokens=8))
    plan, _ = run_step(sched, cm)
    kinds = [(it.seq.seq_id, it.n_tokens) for it in plan.items]
    assert kinds == [(0, 1), (1, 9)]             # one decoded token beside a 9-token portion: budget 10
    plan, _ = run_step(sched, cm)
    assert [(it.seq.seq_id, it.n_tokens) for it in plan.items] == [(0, 1), (1, 9)]
    plan, _ = run_step(sched, cm)
    assert [(it.seq.seq_id, it.n_tokens, it.samples) for it in plan.items] == [(0, 1, True), (1, 2, True)]


def test_chunk_size_and_batch_limits():
    sched, cm = make(max_num_batched_tokens=64, max_num_seqs_in_batch=2, engine_prefill_chunk_size=5)
    for i in range(3):
        sched.add(seq(i, 12))
    plan, _ = run_step(sched, cm)
    assert [(it.seq.seq_id, it.n_tokens) for it in plan.items] == [(0, 5), (1, 5)]   # two portions a step
    assert len(sched.waiting) == 1


def test_finish_on_eos_max_tokens_and_ignore_eos():
    sched, cm = make()
    sched.add(seq(0, 3, max_tokens=3))
    sched.add(seq(1, 3, max_tokens=3, ignore_eos=True))
    sched.add(seq(2, 3, max_tokens=5, eos_token_ids=[5]))
    _, fin = run_step(sched, cm, tokens=[99, 99, 5])
    assert sorted((s.seq_id, s.finish_reason) for s in fin) == [(0, "stop"), (2, "stop")]
    _, fin = run_step(sched, cm, tokens=[99])
    assert fin == []
    _, fin = run_step(sched, cm, tokens=[1])
    assert [(s.seq_id, s.finish_reason, s.output_ids) for s in fin] == [(1, "length", [99, 99, 1])]
    assert sched.is_finished() and cm.free_pages() == 64 and cm.free_rows == cm.max_rows
    cm.check()


def test_forced_tokens_replace_samples():
    sched, cm = make()
    sched.add(seq(0, 2, max_tokens=3, ignore_eos=True, benchmark_forced_token_ids=(11, 12, 13)))
    for _ in range(3):
        _, fin = run_step(sched, cm)
    assert fin[0].output_ids == [11, 12, 13]


def test_admission_waits_for_whole_prompt_and_is_first_come_first_served():
    sched, cm = make(num_pages=8, page_size=4, max_num_batched_tokens=8)
    sched.add(seq(0, 20, max_tokens=2))          # 21 tokens -> 6 pages
    sched.add(seq(1, 9, max_tokens=2))           # 10 tokens -> 3 pages: does not fit beside request 0
    plan, _ = run_step(sched, cm)
    assert [it.seq.seq_id for it in plan.items] == [0] and len(sched.waiting) == 1
    for _ in range(3):
        plan, fin = run_step(sched, cm)
        assert all(it.seq.seq_id == 0 for it in plan.items)
    assert [s.seq_id for s in fin] == [0]
    plan, _ = run_step(sched, cm)
    assert [it.seq.seq_id for it in plan.items] == [1]


def test_out_of_pages_preempts_the_last_admitted_and_recomputes():
    sched, cm = make(num_pages=4, page_size=4, max_num_batched_tokens=64, decode_reservation_tokens=0)
    sched.add(seq(0, 6, max_tokens=6, ignore_eos=True))     # 7 tokens -> 2 pages at admission
    sched.add(seq(1, 6, max_tokens=6, ignore_eos=True))
    run_step(sched, cm)                                      # both prefill: 4 pages held, lengths 6
    run_step(sched, cm)                                      # lengths 7
    plan, _ = run_step(sched, cm)                            # lengths 8: pages full
    assert not plan.preempted
    plan, _ = run_step(sched, cm)                            # both need a third page: none free
    assert [s.seq_id for s in plan.preempted] == [1]
    assert [it.seq.seq_id for it in plan.items] == [0]
    victim = plan.preempted[0]
    assert victim.num_computed == 0 and victim.output_ids == [7, 7, 7] and sched.waiting[0] is victim
    done = {}
    for _ in range(40):
        if sched.is_finished():
            break
        plan, fin = run_step(sched, cm)
        for it in plan.items:
            if it.seq is victim and it.start == 0:
                assert it.n_tokens == 9 and it.samples   # prompt + produced tokens prefilled again as one
        for s in fin:
            done[s.seq_id] = s
    assert sorted(done) == [0, 1] and all(len(s.output_ids) == 6 for s in done.values())
    assert sched.num_preemptions >= 1 and cm.free_pages() == 4
    cm.check()


def test_a_request_too_large_for_the_cache_is_an_error_not_a_loop():
    sched, cm = make(num_pages=2, page_size=4)
    with pytest.raises(ValueError, match="does not fit"):
        sched.add(seq(0, 12))
    sched.add(seq(1, 6, max_tokens=8, ignore_eos=True))
    run_step(sched, cm)
    run_step(sched, cm)
    with pytest.raises(RuntimeError, match="too small"):
        for _ in range(4):
            run_step(sched, cm)
    with pytest.raises(ValueError, match="max_model_len"):
        sched.add(seq(2, 250, max_tokens=100))


def test_abort_frees_everything():
    sched, cm = make()
    sched.add(seq(0, 5))
    sched.add(seq(1, 5))
    run_step(sched, cm)
    assert sched.abort(0) and not sched.abort(42)
    assert cm.free_rows == cm.max_rows - 1
    sched.add(seq(2, 5))
    assert sched.abort(2)                # still waiting
    while not sched.is_finished():
        run_step(sched, cm)
    assert cm.free_pages() == 64
    cm.check()


def test_a_failed_step_ends_its_requests_and_frees_them():
    sched, cm = make(num_pages=16, max_num_batched_tokens=64)
    sched.add(seq(0, 5, max_tokens=8))
    sched.add(seq(1, 6, max_tokens=8))
    run_step(sched, cm)
    plan = sched.schedule()                      # a decode step whose result never arrives
    for it in plan.items:
        cm.reserve(it.seq.seq_id, it.n_tokens)
        cm.commit(it.seq.seq_id, it.n_tokens)
    ended = sched.fail(plan, "error")
    assert [s.seq_id for s in ended] == [0, 1] and all(s.finish_reason == "error" for s in ended)
    assert sched.is_finished() and cm.free_pages() == 16 and cm.free_rows == cm.max_rows
    cm.check()
    assert sched.fail(plan) == []                # nothing of it runs any more


def test_max_decoding_seqs_blocks_new_prompts():
    sched, cm = make(max_num_seqs_in_batch=4, max_decoding_seqs=1)
    sched.add(seq(0, 3, max_tokens=3, ignore_eos=True))
    sched.add(seq(1, 3, max_tokens=3, ignore_eos=True))
    plan, _ = run_step(sched, cm)
    assert [it.seq.seq_id for it in plan.items] == [0, 1]     # nothing decodes yet
    sched.add(seq(2, 3, max_tokens=3, ignore_eos=True))
    plan, _ = run_step(sched, cm)
    assert [it.seq.seq_id for it in plan.items] == [0]        # one decode a step, no new prompt meanwhile


@pytest.mark.parametrize("seed", list(range(12)))
def test_random_workloads_finish_every_request_and_leak_nothing(seed):
    """Random prompt lengths, output lengths, arrival times, aborts, cache sizes and budgets:
    every step stays inside its budgets and continues each request where it stood, every request
    ends with the tokens it asked for (or aborted), and all pages and rows come back."""
    import random
    rng = random.Random(seed)
    page = rng.choice([1, 2, 4, 8])
    budget = rng.choice([4, 8, 16, 64])
    pages = rng.randint(12, 40) * (8 // page)
    sched, cm = make(num_pages=pages, page_size=page, max_model_len=pages * page,
                     max_num_batched_tokens=budget, max_num_seqs_in_batch=rng.choice([1, 2, 4]),
                     max_num_seqs_in_gpu=rng.choice([2, 4, 8]), max_decoding_seqs=rng.choice([2, 4, 8]),
                     engine_prefill_chunk_size=rng.choice([3, 8, 64]),
                     decode_reservation_tokens=rng.choice([0, 4]))
    todo = [seq(i, rng.randint(1, 30), max_tokens=rng.randint(1, 12), ignore_eos=True) for i in range(20)]
    want = {s.seq_id: s.params.max_tokens for s in todo}
    aborted, done = set(), {}
    pending = list(todo)
    for step in range(3000):
        for _ in range(rng.randint(0, 2)):
            if pending:
                sched.add(pending.pop(0))
        if rng.random() < 0.05 and (sched.running or sched.waiting):
            victim = rng.choice(list(sched.running) + list(sched.waiting))
            assert sched.abort(victim.seq_id)
            aborted.add(victim.seq_id)
        if sched.is_finished():
            if not pending:
                break
            continue
        plan, fin = run_step(sched, cm)
        assert 0 < plan.num_tokens <= budget
        ids = [it.seq.seq_id for it in plan.items]
        assert len(ids) == len(set(ids))
        for it in plan.items:
            # a portion starts where the request stood before this step, and samples only at its end
            assert it.start == it.seq.num_computed - it.n_tokens or it.seq.status.name == "FINISHED"
            assert it.n_tokens >= 1
        for s in fin:
            done[s.seq_id] = s
        cm.check()
    else:
        raise AssertionError("the workload did not finish")
    assert set(done) | aborted == set(want)
    for sid, s in done.items():
        assert len(s.output_ids) == want[sid] and s.finish_reason == "length"
    assert cm.free_pages() == pages and cm.free_rows == sched.config.max_num_seqs_in_gpu
    cm.check()
