"""CPU: the host side of the multi-GPU world -- the ring schedule of the key / value exchange, the
launch plan of the chunked attention (which key tiles a launch may read once which ring steps
have landed), the bounded rendezvous, and the behaviour when a rank never shows up. The ranks are
threads or processes on CPU; the transport is host memory or gloo. No GPU, no NCCL, no kernel."""
import ctypes as C
import os
import socket
import time

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


@pytest.fixture(scope="module")
def lib():
    from diffusion_compiler_b200 import _lib, build
    build.build()
    return _lib.lib()


def _plan(lib, rank, size, tiles, groups=()):
    cap = 16
    ranges = (C.c_uint32 * (4 * cap))()
    first = (C.c_int32 * cap)()
    count = (C.c_int32 * cap)()
    n = C.c_int32(0)
    g = (C.c_int32 * max(1, len(groups)))(*groups)
    rc = lib.difb200_world_plan(rank, size, tiles, g, len(groups), ranges, first, count, cap, C.byref(n))
    if rc != 0:
        raise ValueError(lib.difb200_last_error().decode())
    return [dict(ranges=[(ranges[4 * i], ranges[4 * i + 1]), (ranges[4 * i + 2], ranges[4 * i + 3])],
                 first=first[i], steps=count[i]) for i in range(n.value)]


@pytest.mark.parametrize("size,groups", [(1, ()), (2, ()), (4, ()), (8, ()), (8, (1, 3, 4)), (8, (1, 1, 1, 1, 1, 1, 1, 1)),
                                         (5, (2, 3))])
def test_launch_plan_covers_every_slice_once_and_only_after_it_landed(lib, size, groups):
    tiles = 33
    for rank in range(size):
        plan = _plan(lib, rank, size, tiles, groups)
        seen, step = [], 0
        for launch in plan:
            assert launch["first"] == step
            step += launch["steps"]
            # slices this launch may read: those of ring steps launch.first .. first + steps - 1
            allowed = {((rank - s) % size) for s in range(launch["first"], launch["first"] + launch["steps"])}
            covered = []
            for begin, count in launch["ranges"]:
                assert begin % tiles == 0 and count % tiles == 0
                covered += list(range(begin // tiles, (begin + count) // tiles))
            assert set(covered) == allowed and len(covered) == len(allowed)
            seen += covered
        assert step == size and sorted(seen) == list(range(size))
        if plan[0]["steps"] == 1:
            assert plan[0]["ranges"][0] == (rank * tiles, tiles)  # the own slice comes first
    if not groups and size == 8:
        assert [l["steps"] for l in _plan(lib, 0, 8, tiles)] == [1, 7]


def test_launch_plan_rejects_bad_groupings(lib):
    for bad in ((1, 2), (0, 4), (5,)):
        with pytest.raises(ValueError):
            _plan(lib, 0, 4, 8, bad)


@pytest.mark.parametrize("size", [1, 2, 3, 8])
def test_ring_exchange_reassembles_every_buffer_on_every_rank(lib, size):
    assert lib.difb200_world_selftest_fake(size, -1, 5000) == 0, lib.difb200_last_error().decode()


def test_ring_exchange_reports_a_rank_that_never_joins(lib):
    """Rank 2 of 4 is absent from the start: every other rank must return an execution error by
    the deadline instead of waiting forever (the failure is made on the host; nothing hangs)."""
    t0 = time.time()
    assert lib.difb200_world_selftest_fake(4, 2, 300) == 0, lib.difb200_last_error().decode()
    assert time.time() - t0 < 5.0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rendezvous_worker(rank, size, directory, absent, out_dir):
    from diffusion_compiler_b200 import _lib
    lib = _lib.lib()
    if rank == absent:
        return  # this rank leaves before it ever checks in
    ident = (C.c_uint8 * 128)(*([rank + 1] * 128))  # rank 0 publishes 1,1,1,...
    t0 = time.time()
    rc = lib.difb200_world_rendezvous(directory.encode(), rank, size, ident, 3000 if absent >= 0 else 20000)  # 3 s: the ranks start seconds apart
    with open(os.path.join(out_dir, "r%d" % rank), "w") as f:
        f.write("%d %d %.3f %s" % (rc, ident[0], time.time() - t0, lib.difb200_last_error().decode()))


def test_rendezvous_hands_out_the_id_and_is_bounded(tmp_path):
    good, out = tmp_path / "good", tmp_path / "out"
    good.mkdir(), out.mkdir()
    mp.spawn(_rendezvous_worker, args=(3, str(good), -1, str(out)), nprocs=3, join=True)
    for r in range(3):
        rc, first, _, _ = open(out / ("r%d" % r)).read().split(" ", 3)
        assert (int(rc), int(first)) == (0, 1)  # everyone holds rank 0's id
    lost, out2 = tmp_path / "lost", tmp_path / "out2"
    lost.mkdir(), out2.mkdir()
    mp.spawn(_rendezvous_worker, args=(3, str(lost), 1, str(out2)), nprocs=3, join=True)
    for r in (0, 2):
        rc, _, seconds, text = open(out2 / ("r%d" % r)).read().split(" ", 3)
        assert int(rc) == 5 and float(seconds) < 10.0 and "rank 1 of 3 did not arrive" in text


def _gloo_ring_worker(rank, size, port, out_dir):
    """The ring schedule and the launch plan with gloo as the transport: after every step each
    rank checks that exactly the slices its next launch is allowed to read are in place."""
    from diffusion_compiler_b200 import _lib
    lib = _lib.lib()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=size)
    try:
        tiles, width = 2, 16
        rows = tiles * 128
        g = torch.Generator().manual_seed(0)
        full = torch.randint(-128, 127, (size * rows, width), generator=g, dtype=torch.int8)
        mine = torch.zeros_like(full)
        mine[rank * rows:(rank + 1) * rows] = full[rank * rows:(rank + 1) * rows]
        plan = _plan(lib, rank, size, tiles)
        ok = True
        landed = {rank}
        step = 1
        for launch in plan:
            while step < launch["first"] + launch["steps"]:
                if step > 0:
                    to, frm = (rank + step) % size, (rank - step) % size
                    ops = [dist.P2POp(dist.isend, mine[rank * rows:(rank + 1) * rows], to),
                           dist.P2POp(dist.irecv, mine[frm * rows:(frm + 1) * rows], frm)]
                    for w in dist.batch_isend_irecv(ops):
                        w.wait()
                    landed.add(frm)
                step += 1
            for begin, count in launch["ranges"]:
                lo, hi = begin * 128, (begin + count) * 128
                ok = ok and torch.equal(mine[lo:hi], full[lo:hi])
                ok = ok and all((t // tiles) in landed for t in range(begin, begin + count))
        ok = ok and torch.equal(mine, full)
        with open(os.path.join(out_dir, "rank%d" % rank), "w") as f:
            f.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("size", [2, 4])
def test_ring_schedule_over_gloo_feeds_the_launch_plan(tmp_path, size):
    mp.spawn(_gloo_ring_worker, args=(size, _free_port(), str(tmp_path)), nprocs=size, join=True)
    for r in range(size):
        assert open(os.path.join(str(tmp_path), "rank%d" % r)).read() == "ok"
