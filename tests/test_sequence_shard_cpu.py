"""CPU: the token partition of the sharded block -- slice bounds and padding masks. The exchange
schedule and the launch plan of the multi-GPU path are covered in tests/test_world_cpu.py."""
import pytest

from diffusion_compiler_b200.sequence_shard import ShardPlan


def test_shard_plan_even_and_padded():
    p = ShardPlan.make(33272, 8)
    assert p.slice_len == 4159 and p.padded_tokens == 33272 and p.key_valid() is None
    assert [p.bounds(r) for r in (0, 7)] == [(0, 4159), (29113, 33272)]
    p = ShardPlan.make(10, 4)  # 3,3,3,1 real tokens in slices of 3
    assert p.slice_len == 3 and p.padded_tokens == 12
    assert [p.local_tokens(r) for r in range(4)] == [3, 3, 3, 1]
    assert p.key_valid().ravel().tolist() == [1] * 10 + [0, 0]
    p = ShardPlan.make(5, 8)  # more ranks than some slices can fill
    assert sum(p.local_tokens(r) for r in range(8)) == 5
    assert int(p.key_valid().sum()) == 5
    with pytest.raises(ValueError):
        ShardPlan.make(0, 2)
