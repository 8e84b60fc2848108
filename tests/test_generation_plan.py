"""The generation loop's decisions, driven by a fake sampler (no GPU)."""
import pytest

from agave_b200.engine.generate import CONTEXT, LENGTH, STOP, GenerationPlan


def drive(plan, next_token):
    """Run the plan to the end; next_token(request, step) gives the sampled id.
    Returns the order in which batches formed and the number of steps each ran."""
    batches = []
    while True:
        batch = plan.next_batch()
        if not batch:
            break
        steps = 0
        while plan.live():
            live = plan.live()
            plan.accept({r.index: next_token(r, len(r.output)) for r in live})
            steps += 1
        batches.append(([r.index for r in batch], steps))
    return batches


def test_stop_token_ends_early_and_is_not_returned():
    plan = GenerationPlan([[5, 6], [7], [8, 9, 10]], 6, [1], max_batch=8, max_tokens=4096,
                          max_seq_len=128)
    stops_at = {0: 2, 1: 99, 2: 0}
    batches = drive(plan, lambda r, s: 1 if s == stops_at[r.index] else 40 + s)
    assert plan.outputs() == [[40, 41], [40, 41, 42, 43, 44, 45], []]
    assert [r.finish_reason for r in plan.requests] == [STOP, LENGTH, STOP]
    assert batches == [([0, 1, 2], 6)]


def test_batches_follow_each_other_when_slots_run_out():
    prompts = [[3] * n for n in (5, 11, 17, 4, 9)]
    plan = GenerationPlan(prompts, 3, [], max_batch=2, max_tokens=4096, max_seq_len=128)
    batches = drive(plan, lambda r, s: 50)
    assert [b for b, _ in batches] == [[0, 1], [2, 3], [4]]
    assert all(len(o) == 3 for o in plan.outputs()) and plan.finished


def test_token_budget_limits_a_batch():
    # each request may come to hold 64 positions: two fit into 128 tokens
    prompts = [[3] * 10] * 5
    plan = GenerationPlan(prompts, 20, [], max_batch=8, max_tokens=128, max_seq_len=128)
    batches = drive(plan, lambda r, s: 50)
    assert [b for b, _ in batches] == [[0, 1], [2, 3], [4]]


def test_cache_end_clamps_generation():
    plan = GenerationPlan([[3] * 60], 100, [], max_batch=4, max_tokens=64, max_seq_len=64)
    drive(plan, lambda r, s: 50)
    # 60 prompt positions + 4 fed-back tokens fill 64; one more token is sampled, not stored
    assert len(plan.outputs()[0]) == 5
    assert plan.requests[0].finish_reason == CONTEXT


def test_nothing_joins_a_running_batch_and_zero_new_tokens():
    plan = GenerationPlan([[3], [4]], 2, [], max_batch=1, max_tokens=4096, max_seq_len=64)
    assert [r.index for r in plan.next_batch()] == [0]
    with pytest.raises(RuntimeError):
        plan.next_batch()
    plan2 = GenerationPlan([[3], [4]], 0, [], max_batch=4, max_tokens=4096, max_seq_len=64)
    assert plan2.next_batch() == [] and plan2.outputs() == [[], []]


def test_bad_prompts():
    with pytest.raises(ValueError):
        GenerationPlan([[]], 4, [], 4, 4096, 64)
    with pytest.raises(ValueError):
        GenerationPlan([[1] * 65], 4, [], 4, 4096, 64)
