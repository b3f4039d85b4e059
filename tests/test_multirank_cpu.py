"""The N > 1 host logic (batch slices, max-over-ranks timing, gather in rank order) at world size 2 on gloo."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from neoml_b200 import sharding


def test_slices_cover_the_batch_exactly():
    for total in (0, 1, 7, 256, 1000, 1023):
        for world in (1, 2, 3, 4, 8):
            spans = [sharding.image_slice(total, world, r) for r in range(world)]
            assert spans[0][0] == 0
            for (s0, c0), (s1, _) in zip(spans, spans[1:]):
                assert s0 + c0 == s1
            assert spans[-1][0] + spans[-1][1] == total
            counts = [c for _, c in spans]
            assert max(counts) - min(counts) <= 1
    with pytest.raises(ValueError):
        sharding.image_slice(8, 2, 2)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, total: int, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        start, count = sharding.image_slice(total, world, rank)
        counts = [sharding.image_slice(total, world, r)[1] for r in range(world)]
        # the "result" of image i is (i, i*i): a stand-in for (arg-max, probability row) that makes misplaced rows visible
        ids = torch.arange(start, start + count, dtype=torch.int64)
        local = torch.stack([ids, ids * ids], dim=1)
        gathered = sharding.gather_by_rank(local, counts)
        slow = [10.0 + rank, 5.0 - rank]
        mx = sharding.max_over_ranks(slow)
        sm = sharding.sum_over_ranks([float(count)])
        out[rank] = (gathered.tolist(), mx, sm, sharding.whole_job_throughput(sm[0], mx[0]))
    finally:
        dist.destroy_process_group()


def test_two_ranks_on_gloo():
    world, total = 2, 7
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_rank_main, args=(world, _free_port(), total, out), nprocs=world, join=True)
    want = [[i, i * i] for i in range(total)]
    for rank in range(world):
        gathered, mx, sm, thr = out[rank]
        assert gathered == want                      # rank order, no gaps, no duplicates, ragged split (4 + 3)
        assert mx == [11.0, 5.0]                     # slowest rank per entry
        assert sm == [float(total)]
        assert thr == pytest.approx(total / 11.0e-3)
