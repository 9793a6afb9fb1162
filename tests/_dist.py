"""Spawn helper for multi-process tests: one process per rank, rendezvous on 127.0.0.1."""
import os
import socket
import sys
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, use_cuda, fn, args):
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world)
    if use_cuda:
        torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        fn(rank, world, *args)
        if use_cuda:
            torch.cuda.synchronize()
        dist.barrier()
    except Exception:
        traceback.print_exc()
        raise
    finally:
        dist.destroy_process_group()


def run_distributed(fn, world, *args, use_cuda=True):
    """Run fn(rank, world, *args) in `world` processes; raises if any rank fails."""
    mp.spawn(_entry, args=(world, free_port(), use_cuda, fn, args), nprocs=world, join=True)
