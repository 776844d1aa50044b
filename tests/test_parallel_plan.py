"""Shard planning (host logic, no GPU)."""
import pytest


def test_shard_plan_covers_everything_once():
    from oxibonsai_b200.parallel.tp import shard_plan
    for tp in (1, 2, 4, 8):
        plan = shard_plan(32, 8, 12288, 151936, tp)
        assert plan[0].heads[0] == 0 and plan[-1].heads[1] == 32 and plan[-1].kv_heads[1] == 8
        assert plan[-1].inter_blocks[1] == 96 and plan[-1].vocab_rows[1] == 151936
        for a, b in zip(plan, plan[1:]):
            assert a.heads[1] == b.heads[0] and a.inter_blocks[1] == b.inter_blocks[0] and a.vocab_rows[1] == b.vocab_rows[0]
    # 9728 = 76 blocks does not divide by 8: block counts differ by at most one
    plan = shard_plan(32, 8, 9728, 151936, 8)
    sizes = [b - a for a, b in (p.inter_blocks for p in plan)]
    assert sum(sizes) == 76 and max(sizes) - min(sizes) == 1
    with pytest.raises(ValueError):
        shard_plan(32, 8, 12288, 151936, 3)
