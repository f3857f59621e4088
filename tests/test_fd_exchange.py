"""File-descriptor hand-over between processes (the transport of VMM arena and multicast handles), no GPU."""

import os
import uuid

import torch.distributed as dist

from dist_utils import run_distributed


def _worker(rank, world, tag):
    from etha_b200.parallel.arena import exchange_fds

    r, w = os.pipe()
    r2, w2 = os.pipe()
    mine = [w] + ([w2] if rank == 0 else [])
    got = exchange_fds(rank, list(range(world)), mine, tag, dist.barrier)
    assert sorted(got) == [p for p in range(world) if p != rank]
    for peer, fds in got.items():
        assert len(fds) == (2 if peer == 0 else 1)
        os.write(fds[0], bytes([rank]))
        for fd in fds:
            os.close(fd)
    dist.barrier()
    data = os.read(r, 16)
    assert sorted(data) == [p for p in range(world) if p != rank]


def test_all_to_all_fd_exchange():
    run_distributed(_worker, 3, uuid.uuid4().hex[:8])
