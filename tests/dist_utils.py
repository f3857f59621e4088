"""Helpers to run a function on N gloo ranks on this machine."""

import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world_size, port, fn, args, backend):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world_size)
    torch.set_num_threads(1)
    dist.init_process_group(backend=backend, rank=rank, world_size=world_size)
    try:
        fn(rank, world_size, *args)
        dist.barrier()
    except Exception:
        traceback.print_exc()
        raise
    finally:
        dist.destroy_process_group()


def run_distributed(fn, world_size, *args, backend="gloo"):
    """Spawn `world_size` ranks running `fn(rank, world_size, *args)`; raises if any rank fails."""
    mp.spawn(_entry, args=(world_size, free_port(), fn, args, backend), nprocs=world_size, join=True)
