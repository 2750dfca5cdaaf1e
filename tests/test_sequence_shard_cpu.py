"""CPU: the host-side logic of the token-sharded multi-GPU path -- shard bounds, padding masks and
the in-place all-gather of the K/V buffers -- with two gloo ranks (no GPU, no kernels)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from diffusion_compiler_b200.sequence_shard import GatherBuffers, ShardPlan


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


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, tokens, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        KV, D = 2, 8
        plan = ShardPlan.make(tokens, world)
        g = torch.Generator().manual_seed(0)
        full_k = torch.randint(-127, 128, (tokens, KV, D), generator=g, dtype=torch.int8)
        full_s = torch.rand((tokens, KV), generator=g)
        full_v = torch.randn((tokens, KV, D), generator=g).to(torch.bfloat16)
        gb = GatherBuffers(plan, rank, KV, D, "cpu")
        lo, hi = plan.bounds(rank)
        n = hi - lo
        gb.local(gb.k8)[:n] = full_k[lo:hi]  # what the K quantiser / V projection would write
        gb.local(gb.ks)[:n] = full_s[lo:hi]
        gb.local(gb.v)[:n] = full_v[lo:hi]
        gb.all_gather()
        valid = plan.key_valid()
        keep = torch.ones(plan.padded_tokens, dtype=torch.bool) if valid is None else valid.ravel().bool()
        ok = (torch.equal(gb.k8[keep], full_k) and torch.equal(gb.ks[keep], full_s)
              and torch.equal(gb.v[keep].view(torch.int16), full_v.view(torch.int16)))
        with open(os.path.join(result_dir, "rank%d" % rank), "w") as f:
            f.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("tokens", [64, 37])
def test_two_rank_gather_reassembles_the_sequence(tmp_path, tokens):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), tokens, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(os.path.join(str(tmp_path), "rank%d" % r)).read() == "ok"
