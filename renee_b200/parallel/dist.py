"""Process bootstrap: one process per GPU, ``torch.distributed`` for rendezvous and control.

The reference spawns one process per local GPU with ``mp.spawn`` and joins a NCCL group through a
``tcp://`` URL; ``--world-size`` counts nodes and is multiplied by the local GPU count, ``--rank`` is
the node rank (main.py:29-37, 263-269).  Here the same flags are honoured, and a ``torchrun``
environment (``RANK``/``WORLD_SIZE``/``LOCAL_RANK``/``MASTER_ADDR``/``MASTER_PORT``) is accepted as
well.  CPU runs use the ``gloo`` backend so the whole control path is testable without a GPU.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class DistContext:
    rank: int = 0
    world_size: int = 1
    local_rank: int = 0
    device: torch.device = torch.device("cpu")
    backend: str | None = None

    @property
    def is_distributed(self) -> bool:
        return self.world_size > 1

    @property
    def is_main(self) -> bool:
        return self.rank == 0

    def barrier(self) -> None:
        if self.is_distributed:
            dist.barrier()


def env_world() -> tuple[int, int, int] | None:
    """(rank, world, local_rank) from a torchrun-style environment, else ``None``."""
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        return int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    return None


def init_distributed(rank: int | None = None, world_size: int | None = None, local_rank: int | None = None,
                     init_method: str | None = None, device: str | None = None,
                     timeout_s: float = 600.0) -> DistContext:
    env = env_world()
    if rank is None and env is not None:
        rank, world_size, local_rank = env
    rank = 0 if rank is None else rank
    world_size = 1 if world_size is None else world_size
    local_rank = (rank if local_rank is None else local_rank)
    use_cuda = torch.cuda.is_available() and device != "cpu"
    if use_cuda:
        dev = torch.device("cuda", local_rank % max(1, torch.cuda.device_count()))
        torch.cuda.set_device(dev)
    else:
        dev = torch.device("cpu")
    backend = None
    if world_size > 1:
        backend = "nccl" if use_cuda else "gloo"
        if not dist.is_initialized():
            kwargs = dict(backend=backend, rank=rank, world_size=world_size,
                          timeout=datetime.timedelta(seconds=timeout_s))
            if init_method is None and "MASTER_ADDR" not in os.environ:
                os.environ["MASTER_ADDR"] = "127.0.0.1"
                os.environ.setdefault("MASTER_PORT", "23456")
            if init_method is not None:
                kwargs["init_method"] = init_method
            if use_cuda:
                kwargs["device_id"] = dev
            dist.init_process_group(**kwargs)
    return DistContext(rank, world_size, local_rank, dev, backend)


def shutdown() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()
